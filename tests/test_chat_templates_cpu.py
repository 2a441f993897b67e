"""Jinja chat templates: every shipped template renders, and the generation blocks give the assistant-only mask."""
import pytest

from loongforge_b200.data import chat_template as CT

MSGS = [{"role": "system", "content": "Be brief."},
        {"role": "user", "content": "What is 2+2?"},
        {"role": "assistant", "content": "<think>\nadd\n</think>\n\n4"},
        {"role": "user", "content": "Weather in Paris?"},
        {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "weather", "arguments": {"city": "Paris"}}}]},
        {"role": "tool", "content": "sunny"},
        {"role": "assistant", "content": "It is sunny.", "reasoning_content": "tool said sunny"}]
TOOLS = [{"type": "function", "function": {"name": "weather", "parameters": {"type": "object"}}}]
JINJA = [n for n in CT.list_templates() if n.endswith("_training")]


def test_eighteen_jinja_templates_are_listed():
    assert len(JINJA) == 18 and "chatml" in CT.list_templates()


@pytest.mark.parametrize("name", JINJA)
def test_template_renders_with_assistant_only_targets(name):
    tpl = CT.get_template(name)
    plain = [m for m in MSGS if m["role"] != "tool" and not m.get("tool_calls")]
    for msgs, tools in ((plain, None),) + (() if name.startswith(("deepseek_v2", "qwen_chat")) else ((MSGS, TOOLS),)):
        segs = tpl.render(msgs, tools=tools)
        text = "".join(t for t, _ in segs)
        target = "".join(t for t, g in segs if g)
        assert "\x00" not in text
        assert "What is 2+2?" in text and "What is 2+2?" not in target and "Be brief." not in target
        assert "4" in target and sum(1 for _, g in segs if g) == sum(1 for m in msgs if m["role"] == "assistant")
        if tools:
            assert "weather" in target and "sunny" in text and "It is sunny." in target
            assert "sunny</tool_response>" not in target  # tool output is context, not a target


def test_think_modes_and_tool_styles():
    seg = lambda name, msgs=MSGS, tools=TOOLS: "".join(t for t, g in CT.get_template(name).render(msgs, tools=tools) if g)  # noqa: E731
    keep, last = seg("qwen3_hf_training"), seg("qwen3_next_hf_training")
    assert keep.count("<think>") == 3 and "add" in keep
    assert "add" not in last and "tool said sunny" in last  # history reasoning dropped, after the last query kept
    assert seg("qwen3_5_nothink_hf_training").count("<think>\n\n</think>") == 3
    assert "<think>" not in seg("qwen2_5_hf_training") and "add" not in seg("qwen2_5_hf_training")
    assert '{"name": "weather", "arguments": {"city": "Paris"}}' in seg("qwen3_hf_training")
    assert "<function=weather>\n<parameter=city>\nParis\n</parameter>" in seg("qwen3_coder_hf_training")
    assert "<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>" in seg("glm5_2_hf_training")
    assert "functions.weather:0" in seg("kimi_k2_5_training")
    assert "<｜tool▁call▁begin｜>weather<｜tool▁sep｜>" in seg("deepseek_v3_hf_training")


def test_multimodal_parts_become_markers_and_encode_chat_masks():
    msgs = [{"role": "user", "content": [{"type": "image", "image": "a.png"}, {"type": "text", "text": "what?"}]},
            {"role": "assistant", "content": "a cat"}]
    text = "".join(t for t, _ in CT.get_template("qwen3_vl_hf_training").render(msgs))
    assert "<image>what?" in text
    assert "<image>" not in "".join(t for t, _ in CT.get_template("qwen3_hf_training").render(msgs))

    class Tok:
        def tokenize(self, s):
            return [ord(c) for c in s]

    ids, labels = CT.encode_chat(Tok(), msgs, template="qwen3_vl_hf_training")
    tgt = "".join(chr(l) for l in labels if l != -100)
    assert tgt == "a cat<|im_end|>" and len(ids) == len(labels)
    ids2, labels2 = CT.encode_chat(Tok(), [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}],
                                   template="chatml")
    assert "".join(chr(l) for l in labels2 if l != -100) == "yo<|im_end|>\n"
