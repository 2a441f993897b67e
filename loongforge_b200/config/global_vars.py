"""Process-wide singletons: parsed args, composed YAML config, per-component arg copies for VLMs (``args_dict``),
model config, tokenizer and chat template (reference: loongforge/utils/global_vars.py:28-137)."""
from __future__ import annotations

import copy
from typing import Any, Dict, Optional

_G: Dict[str, Any] = {}


def _get(name: str):
    if name not in _G:
        raise RuntimeError(f"{name} is not initialised")
    return _G[name]


def set_args(args) -> None:
    _G["args"] = args


def get_args():
    return _get("args")


def set_yaml_config(cfg) -> None:
    _G["yaml_config"] = cfg


def get_yaml_config():
    return _get("yaml_config")


def set_model_config(cfg) -> None:
    _G["model_config"] = cfg


def get_model_config():
    return _get("model_config")


def set_tokenizer(tok) -> None:
    _G["tokenizer"] = tok


def get_tokenizer():
    return _get("tokenizer")


def set_chat_template(t) -> None:
    _G["chat_template"] = t


def get_chat_template():
    return _G.get("chat_template")


def build_args_dict(args, components: Dict[str, Dict[str, Any]]) -> Dict[str, Any]:
    """One deep copy of the global args per model component (``image_encoder``, ``image_projector``,
    ``foundation``...), each overridden with that component's settings (e.g. its own tensor-parallel size)."""
    out = {}
    for name, overrides in components.items():
        a = copy.deepcopy(args)
        for k, v in overrides.items():
            setattr(a, k, v)
        out[name] = a
    _G["args_dict"] = out
    return out


def get_component_args(name: str):
    return _get("args_dict")[name]


def reset() -> None:
    _G.clear()
