"""Model-family enums and groupings that drive trainer / position-id / loss dispatch (reference:
loongforge/utils/constants.py:72-132)."""
from __future__ import annotations

import enum


class TrainingPhase(str, enum.Enum):
    PRETRAIN = "pretrain"
    SFT = "sft"


class Family(str, enum.Enum):
    LLAMA = "llama"
    QWEN2 = "qwen2"
    QWEN3 = "qwen3"
    QWEN3_5 = "qwen3_5"
    QWEN3_NEXT = "qwen3_next"
    DEEPSEEK = "deepseek"
    DEEPSEEK_V4 = "deepseek_v4"
    GLM = "glm"
    MINIMAX = "minimax"
    MIMO = "mimo"
    INTERNLM = "internlm"
    ERNIE_VL = "ernie4_5_vl"
    QWEN2_VL = "qwen2_vl"
    QWEN3_VL = "qwen3_vl"
    INTERNVL = "internvl"
    LLAVA_OV = "llava_ov"
    KIMI_VL = "kimi_vl"
    MINICPM_V = "minicpm_v"
    WAN = "wan"
    QWEN_IMAGE = "qwen_image"


LANGUAGE_FAMILIES = {Family.LLAMA, Family.QWEN2, Family.QWEN3, Family.QWEN3_5, Family.QWEN3_NEXT, Family.DEEPSEEK,
                     Family.DEEPSEEK_V4, Family.GLM, Family.MINIMAX, Family.MIMO, Family.INTERNLM}
VISION_LANGUAGE_FAMILIES = {Family.QWEN2_VL, Family.QWEN3_VL, Family.INTERNVL, Family.LLAVA_OV, Family.ERNIE_VL,
                            Family.KIMI_VL, Family.MINICPM_V}
DIFFUSION_FAMILIES = {Family.WAN, Family.QWEN_IMAGE}

# which vision encoder / projector a VLM family composes (models/vision.py, models/vision_zoo.py)
VLM_ENCODERS = {
    Family.QWEN2_VL: ("qwen2_vit", "mlp_adapter"),
    Family.QWEN3_VL: ("qwen3_vl_vit", "mlp_adapter"),
    Family.INTERNVL: ("intern_vit", "pixel_shuffle"),
    Family.LLAVA_OV: ("rice_vit", "mlp_adapter"),
    Family.ERNIE_VL: ("ernie_vit", "resampler"),
    Family.KIMI_VL: ("moon_vit", "patch_merger"),
    Family.MINICPM_V: ("minicpm_v_vit", "downsample_mlp"),
}

# M-RoPE position-id variant per family (data/position_ids.py)
POSITION_ID_FUNCS = {Family.QWEN2_VL: "qwen2_vl", Family.QWEN3_VL: "qwen3_vl", Family.QWEN3_5: "qwen3_vl",
                     Family.INTERNVL: "text", Family.ERNIE_VL: "ernie_3d"}

IGNORE_INDEX = -100
