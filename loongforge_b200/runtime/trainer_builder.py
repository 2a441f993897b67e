"""(model family, training phase) -> trainer factory registry
(loongforge/train/trainer_builder.py:13-91)."""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from ..config.constants import LANGUAGE_FAMILIES, VISION_LANGUAGE_FAMILIES

_REGISTRY: Dict[Tuple[str, str], Callable] = {}
# the family groupings of config/constants.py, plus the spellings model YAMLs use for the same families
LLM_FAMILIES = tuple(sorted({f.value for f in LANGUAGE_FAMILIES} | {"qwen"}))
VLM_FAMILIES = tuple(sorted({f.value for f in VISION_LANGUAGE_FAMILIES} | {"qwen2_5_vl"}))


def register_model_trainer(families, phase: str):
    fams = [families] if isinstance(families, str) else list(families)

    def deco(fn):
        for f in fams:
            _REGISTRY[(f, phase)] = fn
        return fn
    return deco


def build_model_trainer(family: str, phase: str, **kw):
    fn = _REGISTRY.get((family, phase))
    if fn is None:
        raise KeyError(f"no trainer registered for family {family!r}, phase {phase!r}; "
                       f"known: {sorted(_REGISTRY)}")
    return fn(**kw)


def _maybe_fsdp(cls, train_cfg):
    if getattr(train_cfg, "use_fsdp", False):
        from .fsdp_trainer import fsdp_variant
        return fsdp_variant(cls)
    return cls


@register_model_trainer(LLM_FAMILIES, "pretrain")
def _llm_pretrain(model_cfg, train_cfg, dims, **kw):
    from .trainer import Trainer
    return _maybe_fsdp(Trainer, train_cfg)(model_cfg, train_cfg, dims, **kw)


@register_model_trainer(LLM_FAMILIES, "sft")
def _llm_sft(model_cfg, train_cfg, dims, **kw):
    from .sft import SFTTrainer
    return _maybe_fsdp(SFTTrainer, train_cfg)(model_cfg, train_cfg, dims, **kw)


@register_model_trainer(VLM_FAMILIES, "pretrain")
@register_model_trainer(VLM_FAMILIES, "sft")
def _vlm(model_cfg, train_cfg, dims, **kw):
    from .vlm import VLMTrainer
    return VLMTrainer(model_cfg, train_cfg, dims, **kw)
