"""Tokenizer front-end in the Megatron tokenizer API (``tokenize``, ``detokenize``, ``vocab_size``,
``eod``, ``pad``), backed by a Hugging Face tokenizer when one is given, with a byte-level fallback
that needs no files (tests, mock data). Vocabulary padding follows
``make_vocab_size_divisible_by x tensor-parallel size``
(loongforge/tokenizer/tokenization_hf.py:14-210, loongforge/tokenizer/tokenizer.py:21-130).
"""
from __future__ import annotations

from typing import List, Optional, Sequence


def padded_vocab_size(vocab_size: int, divisible_by: int = 128, tp: int = 1) -> int:
    mult = divisible_by * tp
    return ((vocab_size + mult - 1) // mult) * mult


class ByteTokenizer:
    """256 byte tokens + <pad>=256, <eod>=257, <bos>=258 and any extra special tokens."""

    def __init__(self, extra_special: Sequence[str] = ()):
        self.special = {"<pad>": 256, "<eod>": 257, "<bos>": 258}
        for s in extra_special:
            self.special.setdefault(s, 256 + len(self.special))
        self.inv_special = {v: k for k, v in self.special.items()}

    @property
    def vocab_size(self):
        return 256 + len(self.special)

    eod = property(lambda self: 257)
    eos = eod
    pad = property(lambda self: 256)
    bos = property(lambda self: 258)

    def tokenize(self, text: str) -> List[int]:
        out, i = [], 0
        specials = sorted(self.special, key=len, reverse=True)
        while i < len(text):
            for s in specials:
                if text.startswith(s, i):
                    out.append(self.special[s])
                    i += len(s)
                    break
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def detokenize(self, ids: Sequence[int]) -> str:
        parts, buf = [], bytearray()
        for t in ids:
            if t < 256:
                buf.append(t)
            else:
                parts.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
                parts.append(self.inv_special.get(int(t), ""))
        parts.append(buf.decode("utf-8", errors="replace"))
        return "".join(parts)

    def convert_tokens_to_ids(self, tok: str) -> int:
        return self.special[tok]


class HFTokenizer:
    """Wrapper around ``transformers.AutoTokenizer`` (loaded from a local path)."""

    def __init__(self, path: str, use_fast: bool = True, additional_special_tokens: Optional[List[str]] = None,
                 chat_template: Optional[str] = None):
        from transformers import AutoTokenizer

        self.tk = AutoTokenizer.from_pretrained(path, use_fast=use_fast, trust_remote_code=False)
        if additional_special_tokens:
            self.tk.add_special_tokens({"additional_special_tokens": list(additional_special_tokens)})
        if self.tk.pad_token_id is None:
            self.tk.pad_token = self.tk.eos_token
        if chat_template:
            self.tk.chat_template = chat_template

    vocab_size = property(lambda self: len(self.tk))
    eod = property(lambda self: self.tk.eos_token_id)
    eos = eod
    pad = property(lambda self: self.tk.pad_token_id)
    bos = property(lambda self: self.tk.bos_token_id)

    def tokenize(self, text: str) -> List[int]:
        return self.tk.encode(text, add_special_tokens=False)

    def detokenize(self, ids) -> str:
        return self.tk.decode(list(ids))

    def convert_tokens_to_ids(self, tok: str) -> int:
        return self.tk.convert_tokens_to_ids(tok)


def build_tokenizer(tokenizer_type: str = "ByteTokenizer", path: Optional[str] = None, **kw):
    if tokenizer_type in ("HFTokenizer", "HuggingFaceTokenizer") and path:
        return HFTokenizer(path, **kw)
    return ByteTokenizer(kw.get("additional_special_tokens") or ())
