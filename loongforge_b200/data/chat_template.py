"""Chat templates for supervised fine-tuning: turn a list of {role, content} messages into token
ids with a loss mask that covers assistant replies only (the reference's template registry,
loongforge/data/chat_template.py, with 18 Jinja templates). Templates here are declarative:
a prefix/suffix per role plus a system default, which covers the ChatML (Qwen), Llama-3,
Llama-2, DeepSeek, InternLM2, Mistral and plain "alpaca" families."""
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


def get_template(name: str) -> ChatTemplate:
    if name not in _TEMPLATES:
        raise KeyError(f"unknown chat template {name!r}; known: {sorted(_TEMPLATES)}")
    return _TEMPLATES[name]


def to_messages(example: Dict, fmt: str = "auto") -> List[Dict[str, str]]:
    """alpaca ({instruction,input,output}), sharegpt ({conversations:[{from,value}]}) and openai
    ({messages:[{role,content}]}) records -> role/content messages."""
    if fmt == "auto":
        fmt = "openai" if "messages" in example else "sharegpt" if "conversations" in example else "alpaca"
    if fmt == "openai":
        return [{"role": m["role"], "content": m["content"]} for m in example["messages"]]
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


def encode_chat(tokenizer, messages, template: str = "chatml", train_on_prompt: bool = False, max_len: Optional[int] = None):
    """-> (input_ids, labels) with labels = -100 on non-target tokens (before the causal shift)."""
    ids: List[int] = []
    labels: List[int] = []
    for text, tgt in get_template(template).render(messages):
        t = tokenizer.tokenize(text)
        ids.extend(t)
        labels.extend(t if (tgt or train_on_prompt) else [-100] * len(t))
    if max_len is not None:
        ids, labels = ids[:max_len], labels[:max_len]
    return ids, labels
