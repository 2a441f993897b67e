"""Chat templates for supervised fine-tuning: turn a list of {role, content} messages into token
ids with a loss mask that covers assistant replies only (the reference's template registry,
loongforge/data/chat_template.py, with 18 Jinja templates). Two kinds of templates live here:
declarative ones (a prefix/suffix per role plus a system default: ChatML, Llama-3, Llama-2, DeepSeek,
InternLM2, Mistral, "alpaca"), and Jinja templates under ``data/chat_templates/*.jinja`` (tool calls, reasoning
blocks, multimodal content parts) in which ``{% generation %} ... {% endgeneration %}`` blocks mark the spans the
model is trained on; `JinjaChatTemplate` turns those marks into the loss mask. ``--chat-template`` takes the name of
either kind or the path of a ``.jinja`` file."""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple


@dataclasses.dataclass
class ChatTemplate:
    name: str
    user: Tuple[str, str]
    assistant: Tuple[str, str]
    system: Tuple[str, str] = ("", "")
    default_system: Optional[str] = None
    bos: str = ""
    generation_prefix: str = ""  # text that precedes the assistant reply and is not trained on

    def render(self, messages: Sequence[Dict[str, str]]) -> List[Tuple[str, bool]]:
        """[(text, is_target)] segments."""
        segs: List[Tuple[str, bool]] = []
        if self.bos:
            segs.append((self.bos, False))
        msgs = list(messages)
        if msgs and msgs[0]["role"] == "system":
            segs.append((self.system[0] + msgs[0]["content"] + self.system[1], False))
            msgs = msgs[1:]
        elif self.default_system is not None:
            segs.append((self.system[0] + self.default_system + self.system[1], False))
        for m in msgs:
            if m["role"] in ("user", "human", "tool", "observation"):
                segs.append((self.user[0] + m["content"] + self.user[1], False))
            elif m["role"] in ("assistant", "gpt"):
                segs.append((self.assistant[0], False))
                segs.append((m["content"] + self.assistant[1], True))
            else:
                raise ValueError(f"unknown role {m['role']!r}")
        return segs


_TEMPLATES: Dict[str, ChatTemplate] = {}


def register_template(t: ChatTemplate):
    _TEMPLATES[t.name] = t
    return t


register_template(ChatTemplate("chatml", ("<|im_start|>user\n", "<|im_end|>\n"), ("<|im_start|>assistant\n", "<|im_end|>\n"),
                               ("<|im_start|>system\n", "<|im_end|>\n")))
register_template(ChatTemplate("qwen", ("<|im_start|>user\n", "<|im_end|>\n"), ("<|im_start|>assistant\n", "<|im_end|>\n"),
                               ("<|im_start|>system\n", "<|im_end|>\n"), default_system="You are a helpful assistant."))
register_template(ChatTemplate("qwen2-vl", ("<|im_start|>user\n", "<|im_end|>\n"), ("<|im_start|>assistant\n", "<|im_end|>\n"),
                               ("<|im_start|>system\n", "<|im_end|>\n"), default_system="You are a helpful assistant."))
register_template(ChatTemplate("llama3", ("<|start_header_id|>user<|end_header_id|>\n\n", "<|eot_id|>"),
                               ("<|start_header_id|>assistant<|end_header_id|>\n\n", "<|eot_id|>"),
                               ("<|start_header_id|>system<|end_header_id|>\n\n", "<|eot_id|>"), bos="<|begin_of_text|>"))
register_template(ChatTemplate("llama2", ("[INST] ", " [/INST]"), (" ", " </s>"), ("<<SYS>>\n", "\n<</SYS>>\n\n"), bos="<s>"))
register_template(ChatTemplate("deepseek", ("<｜User｜>", ""), ("<｜Assistant｜>", "<｜end▁of▁sentence｜>"), ("", ""),
                               bos="<｜begin▁of▁sentence｜>"))
register_template(ChatTemplate("internlm2", ("<|im_start|>user\n", "<|im_end|>\n"), ("<|im_start|>assistant\n", "<|im_end|>\n"),
                               ("<|im_start|>system\n", "<|im_end|>\n"), bos="<s>"))
register_template(ChatTemplate("mistral", ("[INST] ", " [/INST]"), ("", "</s>"), bos="<s>"))
register_template(ChatTemplate("alpaca", ("### Instruction:\n", "\n\n"), ("### Response:\n", "\n\n"),
                               default_system="Below is an instruction that describes a task. Write a response that "
                                              "appropriately completes the request.\n\n"))
register_template(ChatTemplate("empty", ("", ""), ("", "")))


_GEN_OPEN, _GEN_CLOSE = "\x00<gen>\x00", "\x00</gen>\x00"


def _jinja_env(search_dir: str):
    import jinja2
    from jinja2 import nodes
    from jinja2.ext import Extension

    class Generation(Extension):
        """``{% generation %}body{% endgeneration %}``: the body is emitted between two sentinel strings."""
        tags = {"generation"}

        def parse(self, parser):
            lineno = next(parser.stream).lineno
            body = parser.parse_statements(["name:endgeneration"], drop_needle=True)
            return nodes.CallBlock(self.call_method("_mark"), [], [], body).set_lineno(lineno)

        def _mark(self, caller):
            return _GEN_OPEN + caller() + _GEN_CLOSE

    import json
    env = jinja2.Environment(loader=jinja2.FileSystemLoader(search_dir), extensions=[Generation],
                             trim_blocks=True, lstrip_blocks=True, keep_trailing_newline=False)
    env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False, **kw)
    return env


class JinjaChatTemplate:
    """A ``.jinja`` chat template with generation blocks. ``render`` returns the same ``[(text, is_target)]`` segments
    as the declarative templates: text inside a generation block is a target."""

    def __init__(self, path: str):
        import os
        self.path = path
        self.name = os.path.splitext(os.path.basename(path))[0]
        self._tpl = _jinja_env(os.path.dirname(os.path.abspath(path))).get_template(os.path.basename(path))

    def render(self, messages: Sequence[Dict], tools: Optional[List[Dict]] = None,
               add_generation_prompt: bool = False, **kw) -> List[Tuple[str, bool]]:
        text = self._tpl.render(messages=list(messages), tools=tools, add_generation_prompt=add_generation_prompt, **kw)
        segs: List[Tuple[str, bool]] = []
        rest, inside = text, False
        while rest:
            mark = _GEN_CLOSE if inside else _GEN_OPEN
            i = rest.find(mark)
            if i < 0:
                if inside:
                    raise ValueError(f"template {self.name}: generation block not closed")
                segs.append((rest, False))
                break
            if i:
                segs.append((rest[:i], inside))
            rest = rest[i + len(mark):]
            inside = not inside
        return segs


def jinja_template_dir() -> str:
    import os
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "chat_templates")


def list_templates() -> List[str]:
    import os
    jin = [f[:-6] for f in os.listdir(jinja_template_dir()) if f.endswith(".jinja") and not f.startswith("_")]
    return sorted(_TEMPLATES) + sorted(jin)


_JINJA_CACHE: Dict[str, JinjaChatTemplate] = {}


def get_template(name: str):
    """Declarative template by name, Jinja template by file stem (``qwen3_hf_training``) or by path."""
    import os
    if name in _TEMPLATES:
        return _TEMPLATES[name]
    path = name if name.endswith(".jinja") and os.path.isfile(name) else os.path.join(jinja_template_dir(), name + ".jinja")
    if os.path.isfile(path):
        if path not in _JINJA_CACHE:
            _JINJA_CACHE[path] = JinjaChatTemplate(path)
        return _JINJA_CACHE[path]
    raise KeyError(f"unknown chat template {name!r}; known: {list_templates()}")


def to_messages(example: Dict, fmt: str = "auto") -> List[Dict[str, str]]:
    """alpaca ({instruction,input,output}), sharegpt ({conversations:[{from,value}]}) and openai
    ({messages:[{role,content}]}) records -> role/content messages."""
    if fmt == "auto":
        fmt = "openai" if "messages" in example else "sharegpt" if "conversations" in example else "alpaca"
    if fmt == "openai":
        # tool calls, reasoning and multimodal content parts travel with the message (the Jinja templates read them)
        return [dict(m) for m in example["messages"]]
    if fmt == "sharegpt":
        role = {"human": "user", "gpt": "assistant", "system": "system", "user": "user", "assistant": "assistant"}
        return [{"role": role[c["from"]], "content": c["value"]} for c in example["conversations"]]
    msgs = []
    if example.get("system"):
        msgs.append({"role": "system", "content": example["system"]})
    prompt = example.get("instruction", "")
    if example.get("input"):
        prompt = prompt + "\n" + example["input"]
    msgs.append({"role": "user", "content": prompt})
    msgs.append({"role": "assistant", "content": example.get("output", "")})
    return msgs


def encode_chat(tokenizer, messages, template: str = "chatml", train_on_prompt: bool = False, max_len: Optional[int] = None,
                tools: Optional[List[Dict]] = None):
    """-> (input_ids, labels) with labels = -100 on non-target tokens (before the causal shift). Segments are tokenised
    one by one, so the mask boundary is exact whatever the tokenizer merges inside a segment."""
    ids: List[int] = []
    labels: List[int] = []
    tpl = get_template(template)
    segs = tpl.render(messages, tools=tools) if isinstance(tpl, JinjaChatTemplate) else tpl.render(messages)
    for text, tgt in segs:
        t = tokenizer.tokenize(text)
        ids.extend(t)
        labels.extend(t if (tgt or train_on_prompt) else [-100] * len(t))
    if max_len is not None:
        ids, labels = ids[:max_len], labels[:max_len]
    return ids, labels
