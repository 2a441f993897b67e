"""Named record layouts of SFT data (``--sft-dataset NAME ...`` with ``--sft-dataset-config FILE``): which keys of a record
hold the prompt / response / history / messages / tools / images, and how roles are spelled inside a message, mapped to the
role / content messages the chat templates render (reference: loongforge/data/sft_format_utils.py,
sft_supervised_utils.py, configs/data/sft_dataset_config.yaml)."""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict, List, Optional, Tuple

import yaml

DEFAULT_CONFIG = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                              "configs", "data", "sft_dataset_config.yaml")

_TAG_DEFAULTS = dict(role_tag="role", content_tag="content", user_tag="user", assistant_tag="assistant", system_tag="system",
                     tool_tag="tool", observation_tag="observation", function_tag="function_call")


@dataclasses.dataclass
class DatasetFormat:
    name: str
    format: str = "alpaca"                      # alpaca | sharegpt | openai
    columns: Dict[str, str] = dataclasses.field(default_factory=dict)
    tags: Dict[str, str] = dataclasses.field(default_factory=dict)

    def tag(self, key: str) -> str:
        return self.tags.get(key, _TAG_DEFAULTS[key])

    def col(self, key: str, default: Optional[str] = None) -> Optional[str]:
        return self.columns.get(key, default)


def load_dataset_config(path: Optional[str] = None) -> Dict[str, DatasetFormat]:
    path = path or DEFAULT_CONFIG
    with open(path) as f:
        raw = json.load(f) if path.endswith(".json") else yaml.safe_load(f)
    out = {}
    for name, node in (raw or {}).items():
        fmt = node.get("format", node.get("formatting", "alpaca"))
        if fmt not in ("alpaca", "sharegpt", "openai"):
            raise ValueError(f"{path}: data set {name!r} has unknown format {fmt!r}")
        out[name] = DatasetFormat(name, fmt, dict(node.get("columns") or {}), dict(node.get("tags") or {}))
    return out


def resolve_formats(names: List[str], n_files: int, config_path: Optional[str] = None) -> List[DatasetFormat]:
    """One name for all files or one per file."""
    table = load_dataset_config(config_path)
    missing = [n for n in names if n not in table]
    if missing:
        raise KeyError(f"data set name(s) {missing} are not defined in {config_path or DEFAULT_CONFIG}; known: {sorted(table)}")
    if len(names) == 1:
        return [table[names[0]]] * n_files
    if len(names) != n_files:
        raise ValueError(f"{len(names)} data set names for {n_files} data files")
    return [table[n] for n in names]


def _messages(raw: List[dict], f: DatasetFormat) -> List[Dict[str, Any]]:
    role_of = {f.tag("user_tag"): "user", f.tag("assistant_tag"): "assistant", f.tag("system_tag"): "system",
               f.tag("tool_tag"): "tool", f.tag("observation_tag"): "tool", f.tag("function_tag"): "assistant"}
    rk, ck = f.tag("role_tag"), f.tag("content_tag")
    out = []
    for m in raw:
        role = role_of.get(m.get(rk))
        if role is None:
            raise ValueError(f"data set {f.name!r}: unknown role {m.get(rk)!r} (tags: {f.tags})")
        msg = {k: v for k, v in m.items() if k not in (rk, ck)}      # tool_calls, reasoning_content ... travel along
        msg.update(role=role, content=m.get(ck, ""))
        if m.get(rk) == f.tag("function_tag") and isinstance(msg["content"], str):
            try:  # sharegpt function calls are JSON in the content
                call = json.loads(msg["content"])
                msg["tool_calls"] = [{"type": "function", "function": c} for c in (call if isinstance(call, list) else [call])]
                msg["content"] = ""
            except json.JSONDecodeError:
                pass
        out.append(msg)
    return out


def convert(example: Dict[str, Any], f: DatasetFormat) -> Tuple[List[Dict[str, Any]], Optional[list], Optional[list]]:
    """-> (messages, tools, images)."""
    tools = example.get(f.col("tools", "tools"))
    if isinstance(tools, str) and tools.strip():
        tools = json.loads(tools)
    images = example.get(f.col("images")) if f.col("images") else None
    if f.format in ("sharegpt", "openai"):
        msgs = _messages(example[f.col("messages", "messages" if f.format == "openai" else "conversations")], f)
        system = example.get(f.col("system")) if f.col("system") else None
        if system and not (msgs and msgs[0]["role"] == "system"):
            msgs.insert(0, {"role": "system", "content": system})
        return msgs, tools or None, images
    msgs = []
    system = example.get(f.col("system", "system"))
    if system:
        msgs.append({"role": "system", "content": system})
    for turn in example.get(f.col("history", "history")) or []:
        msgs.append({"role": "user", "content": turn[0]})
        msgs.append({"role": "assistant", "content": turn[1]})
    prompt = example.get(f.col("prompt", "instruction"), "") or ""
    query = example.get(f.col("query", "input"), "") or ""
    msgs.append({"role": "user", "content": prompt + ("\n" + query if query else "")})
    msgs.append({"role": "assistant", "content": example.get(f.col("response", "output"), "") or ""})
    return msgs, tools or None, images
