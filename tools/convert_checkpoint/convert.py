"""Offline checkpoint converter: Hugging Face safetensors <-> Megatron-core legacy checkpoints
(``iter_*/mp_rank_{tp:02d}[_{pp:03d}][_{ep:03d}]/model_optim_rng.pt`` + tracker file), with TP / PP /
EP sharding and merging. Same command-line spelling as the reference's tool
(tools/convert_checkpoint/arguments.py:45-258, module_convertor/model.py:250-383,
mcore/mcore_checkpoint.py:520-610).

    python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
        --model_type_custom llama3 --load_ckpt_path <hf dir> --save_ckpt_path <out> \
        --tensor_model_parallel_size 2 --pipeline_model_parallel_size 2 [--safetensors]
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
import sys
from typing import Dict, List, Optional

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from tools.convert_checkpoint import name_maps as nm  # noqa: E402


def parse_args(argv=None):
    p = argparse.ArgumentParser("convert_checkpoint")
    p.add_argument("--load_platform", required=True, choices=["huggingface", "mcore"])
    p.add_argument("--save_platform", required=True, choices=["huggingface", "mcore"])
    p.add_argument("--load_ckpt_path", required=True)
    p.add_argument("--save_ckpt_path", required=True)
    p.add_argument("--model_type_custom", default="llama3")
    p.add_argument("--config_file", default=None, help="model YAML; otherwise config.json of the HF directory is read")
    p.add_argument("--convert_file", default=None,
                   help="conversion descriptor (configs/models/*/ckpt_convert/*.yaml, the `convert_file` key of a model "
                        "YAML): selects the name-map family and side defaults")
    p.add_argument("--safetensors", action="store_true")
    p.add_argument("--torch_dtype", default=None, choices=[None, "float16", "float32", "bfloat16"])
    p.add_argument("--tensor_model_parallel_size", type=int, default=1)
    p.add_argument("--pipeline_model_parallel_size", type=int, default=1)
    p.add_argument("--expert_parallel_size", type=int, default=1)
    p.add_argument("--custom_pipeline_layers", default=None)
    p.add_argument("--make_vocab_size_divisible_by", type=int, default=128)
    p.add_argument("--vocab_size", type=int, default=None)
    p.add_argument("--num_layers", type=int, default=None)
    p.add_argument("--num_attention_heads", type=int, default=None)
    p.add_argument("--num_query_groups", type=int, default=None)
    p.add_argument("--num_experts", type=int, default=None)
    p.add_argument("--language_family", default=None,
                   help="name-map family of the language model inside an InternVL / Kimi-VL composition "
                        "(--model_type_custom internvl | kimi_vl ...), e.g. qwen3, qwen2.5, internlm2.5, deepseek")
    p.add_argument("--vit_num_layers", type=int, default=None, help="vision tower depth (else vision_config.depth)")
    p.add_argument("--vit_num_heads", type=int, default=None, help="vision tower heads (else vision_config.num_heads)")
    p.add_argument("--linear_attention_geometry", default=None,
                   help="key heads,key dim,value heads,value dim of the GatedDeltaNet layers (Qwen3-Next / Qwen3.5 with "
                        "tensor parallelism; else linear_* of config.json)")
    p.add_argument("--no_load_optim", action="store_true")
    p.add_argument("--no_save_optim", action="store_true")
    p.add_argument("--load_lora_ckpt_path", default=None)
    p.add_argument("--lora_alpha", type=int, default=None)
    p.add_argument("--lora_dim", type=int, default=None)
    args = p.parse_args(argv)
    if args.convert_file:
        apply_convert_file(args, args.convert_file)
    return args


def apply_convert_file(args, path: str) -> None:
    """Descriptor keys: ``family`` (name-map family, replaces --model_type_custom), ``huggingface.safetensors``,
    ``mcore.make_vocab_size_divisible_by``. Explicit command-line values win over the descriptor."""
    import yaml

    with open(os.path.expandvars(path)) as f:
        d = yaml.safe_load(f) or {}
    if d.get("family") and args.model_type_custom == "llama3":
        args.model_type_custom = d["family"]
    if (d.get("huggingface") or {}).get("safetensors") and not args.safetensors:
        args.safetensors = True
    div = (d.get("mcore") or {}).get("make_vocab_size_divisible_by")
    if div and args.make_vocab_size_divisible_by == 128:
        args.make_vocab_size_divisible_by = int(div)


def _model_dims(args, hf_dir: Optional[str]):
    cfg = {}
    if hf_dir and os.path.isfile(os.path.join(hf_dir, "config.json")):
        cfg = json.load(open(os.path.join(hf_dir, "config.json")))
    tc = cfg.get("text_config") or cfg.get("llm_config") or cfg  # vision-language configs nest the language model's fields
    L = args.num_layers or tc.get("num_hidden_layers")
    H = args.num_attention_heads or tc.get("num_attention_heads")
    G = args.num_query_groups or tc.get("num_key_value_heads") or H
    V = args.vocab_size or tc.get("vocab_size")
    E = args.num_experts or tc.get("num_experts") or tc.get("n_routed_experts")
    tie = bool(tc.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False)))
    assert L and H, "number of layers / heads unknown: pass --num_layers/--num_attention_heads or provide config.json"
    return L, H, G, V, E, tie, cfg


def load_hf(path: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    out: Dict[str, torch.Tensor] = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        for f in files:
            out.update(load_file(f))
        return out
    for f in sorted(glob.glob(os.path.join(path, "*.bin"))) + sorted(glob.glob(os.path.join(path, "*.pt"))):
        out.update(torch.load(f, map_location="cpu", weights_only=True))
    assert out, f"no weights found in {path}"
    return out


def save_hf(sd: Dict[str, torch.Tensor], path: str, cfg: Optional[dict] = None, shard_bytes: int = 5 << 30):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    shards, cur, size = [], {}, 0
    for k, v in sd.items():
        n = v.numel() * v.element_size()
        if cur and size + n > shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = v.contiguous()
        size += n
    shards.append(cur)
    index = {"metadata": {"total_size": sum(v.numel() * v.element_size() for v in sd.values())}, "weight_map": {}}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors" if len(shards) > 1 else "model.safetensors"
        save_file(sh, os.path.join(path, name), metadata={"format": "pt"})
        for k in sh:
            index["weight_map"][k] = name
    if len(shards) > 1:
        json.dump(index, open(os.path.join(path, "model.safetensors.index.json"), "w"), indent=1)
    if cfg:
        json.dump(cfg, open(os.path.join(path, "config.json"), "w"), indent=1)


def layer_split(L: int, pp: int, custom: Optional[str]) -> List[List[int]]:
    counts = [int(x) for x in custom.split(",")] if custom else [L // pp] * pp
    assert len(counts) == pp and sum(counts) == L, "pipeline layer counts must sum to num_layers"
    out, s = [], 0
    for c in counts:
        out.append(list(range(s, s + c)))
        s += c
    return out


# the language model's layers, optionally under the prefix of a vision-language composition (the encoder's own
# "encoder_model...decoder.layers" are never pipelined and do not match)
_LAYER = re.compile(r"^((?:foundation_model\.)?)decoder\.layers\.(\d+)\.(.*)$")
_EXPERT = re.compile(r"\.experts\.linear_fc[12]\.weight(\d+)$")


def save_mcore(mc: Dict[str, torch.Tensor], path: str, *, tp: int, pp: int, ep: int, num_layers: int,
               num_experts: Optional[int], custom_layers: Optional[str], args_dump: dict, iteration="release"):
    """Legacy per-rank files; layer indices restart at 0 on every pipeline stage, experts are renumbered
    locally on every expert-parallel rank."""
    split = layer_split(num_layers, pp, custom_layers)
    e_local = (num_experts // ep) if num_experts else 0
    release = iteration == "release"
    top = os.path.join(path, "release" if release else f"iter_{int(iteration):07d}")
    for p_rank in range(pp):
        local_of = {g: l for l, g in enumerate(split[p_rank])}
        for t_rank in range(tp):
            for e_rank in range(ep):
                sd = {}
                for k, w in mc.items():
                    m = _LAYER.match(k)
                    if m:
                        g = int(m.group(2))
                        if g not in local_of:
                            continue
                        key = f"{m.group(1)}decoder.layers.{local_of[g]}.{m.group(3)}"
                    else:
                        bare = k[len("foundation_model."):] if k.startswith("foundation_model.") else k
                        # the vision encoder and projector sit on the first stage with the embedding
                        first = bare.startswith(("embedding.", "encoder_model."))
                        # multi-token-prediction layers live on the stage that computes the loss
                        last = bare.startswith(("decoder.final_layernorm", "output_layer", "mtp."))
                        if (first and p_rank != 0) or (last and p_rank != pp - 1):
                            continue
                        key = k
                    em = _EXPERT.search(key)
                    if em:
                        e = int(em.group(1))
                        if not (e_rank * e_local <= e < (e_rank + 1) * e_local):
                            continue
                        key = key[: em.start(1)] + str(e - e_rank * e_local)
                    sd[key] = nm.shard_tp(k, w, t_rank, tp).clone()
                name = f"mp_rank_{t_rank:02d}" + (f"_{p_rank:03d}" if pp > 1 else "") + (f"_{e_rank:03d}" if ep > 1 else "")
                d = os.path.join(top, name)
                os.makedirs(d, exist_ok=True)
                torch.save({"model": sd, "checkpoint_version": 3.0, "iteration": 0 if release else int(iteration),
                            "args": args_dump}, os.path.join(d, "model_optim_rng.pt"))
    with open(os.path.join(path, "latest_checkpointed_iteration.txt"), "w") as f:
        f.write("release" if release else str(iteration))


def load_mcore(path: str, *, num_layers: int, custom_layers: Optional[str]) -> Dict[str, torch.Tensor]:
    tracker = os.path.join(path, "latest_checkpointed_iteration.txt")
    it = open(tracker).read().strip() if os.path.isfile(tracker) else "release"
    top = os.path.join(path, "release" if it == "release" else f"iter_{int(it):07d}")
    dirs = sorted(d for d in os.listdir(top) if d.startswith("mp_rank_"))
    coords = []
    for d in dirs:
        parts = d[len("mp_rank_"):].split("_")
        coords.append((d, [int(x) for x in parts]))
    tp = max(c[1][0] for c in coords) + 1
    extra = max(len(c[1]) for c in coords)
    # the second field is the pipeline rank unless only expert parallelism was used
    sample = torch.load(os.path.join(top, coords[0][0], "model_optim_rng.pt"), map_location="cpu", weights_only=False)
    saved_args = sample.get("args", {}) or {}
    pp = int(saved_args.get("pipeline_model_parallel_size", 1))
    ep = int(saved_args.get("expert_parallel_size", 1))
    split = layer_split(num_layers, pp, custom_layers or saved_args.get("custom_pipeline_layers"))
    pieces: Dict[str, Dict[int, torch.Tensor]] = {}
    for d, c in coords:
        t_rank = c[0]
        p_rank = c[1] if pp > 1 else 0
        e_rank = (c[2] if pp > 1 else c[1]) if ep > 1 else 0
        sd = torch.load(os.path.join(top, d, "model_optim_rng.pt"), map_location="cpu", weights_only=False)["model"]
        e_local = None
        for k, w in sd.items():
            m = _LAYER.match(k)
            key = f"{m.group(1)}decoder.layers.{split[p_rank][int(m.group(2))]}.{m.group(3)}" if m else k
            em = _EXPERT.search(key)
            if em:
                if e_local is None:
                    e_local = 1 + max(int(_EXPERT.search(kk).group(1)) for kk in sd if _EXPERT.search(kk))
                key = key[: em.start(1)] + str(int(em.group(1)) + e_rank * e_local)
            pieces.setdefault(key, {})[t_rank] = w
    return {k: nm.merge_tp(k, [v[t] for t in sorted(v)]) for k, v in pieces.items()}


def merge_lora_into(mc: Dict[str, torch.Tensor], lora_sd: Dict[str, torch.Tensor], alpha: float, dim: int):
    """Fold ``lora_B @ lora_A * alpha/dim`` adapter pairs (keys ``<module>.lora_A`` / ``.lora_B``) into the base weights."""
    scale = alpha / dim
    for k in [k for k in lora_sd if k.endswith(".lora_A")]:
        base = k[: -len(".lora_A")].replace(".base", "") + ".weight"
        if base in mc:
            mc[base] = (mc[base].float() + scale * lora_sd[k[:-1] + "B"].float() @ lora_sd[k].float()).to(mc[base].dtype)


def main(argv=None):
    a = parse_args(argv)
    composite = nm.COMPOSITE_VLM.get(a.model_type_custom)
    if composite and not a.language_family:
        raise SystemExit(f"--model_type_custom {a.model_type_custom} needs --language_family (the language model's name-map family)")
    vlm = a.model_type_custom in nm.VLM_FAMILIES
    fam = nm.FAMILIES[a.language_family if composite else nm.VLM_FAMILIES[a.model_type_custom] if vlm else a.model_type_custom]
    dt = getattr(torch, a.torch_dtype) if a.torch_dtype else None
    hf_dir = a.load_ckpt_path if a.load_platform == "huggingface" else None
    L, H, G, V, E, tie, hf_cfg = _model_dims(a, hf_dir)
    tc = hf_cfg.get("text_config") or hf_cfg.get("llm_config") or hf_cfg
    nm.set_qk_norm_over_all_heads(a.model_type_custom == "minimax")
    if a.linear_attention_geometry:
        nm.set_linear_attention_geometry(*[int(x) for x in a.linear_attention_geometry.split(",")])
    elif tc.get("linear_num_key_heads"):
        nm.set_linear_attention_geometry(tc["linear_num_key_heads"], tc["linear_key_head_dim"],
                                         tc["linear_num_value_heads"], tc["linear_value_head_dim"])
    if a.load_platform == "huggingface":
        hf = load_hf(a.load_ckpt_path)
        mult = a.make_vocab_size_divisible_by * a.tensor_model_parallel_size
        if composite:
            vc = hf_cfg.get("vision_config", {})
            vit = dict(vit_layers=a.vit_num_layers or vc.get("num_hidden_layers") or vc.get("depth"),
                       vit_heads=a.vit_num_heads or vc.get("num_attention_heads") or vc.get("num_heads"))
            V = a.vocab_size or tc.get("vocab_size") or hf["language_model." + fam.hf_prefix + "embed_tokens.weight"].shape[0]
            padded = -(-V // mult) * mult
            mc = nm.composite_vlm_hf_to_mcore(hf, fam, composite, num_layers=L, num_heads=H, num_groups=G, padded_vocab=padded,
                                              num_experts=E, tie_embeddings=tie, **vit)
        elif not vlm:
            V = V or hf[fam.hf_prefix + "embed_tokens.weight"].shape[0]
            padded = -(-V // mult) * mult
        if vlm and not composite:
            vc = hf_cfg.get("vision_config", {})
            vit = dict(vit_layers=a.vit_num_layers or vc.get("depth"), vit_heads=a.vit_num_heads or vc.get("num_heads"))
            lp, _ = nm._vlm_prefixes(hf)
            V = a.vocab_size or hf_cfg.get("vocab_size") or hf[lp + "embed_tokens.weight"].shape[0]
            padded = -(-V // mult) * mult
            mc = nm.vlm_hf_to_mcore(hf, fam, num_layers=L, num_heads=H, num_groups=G, padded_vocab=padded,
                                    num_experts=E, tie_embeddings=tie, **vit)
        elif not composite:
            mc = nm.hf_to_mcore(hf, fam, num_layers=L, num_heads=H, num_groups=G, padded_vocab=padded, num_experts=E,
                                tie_embeddings=tie)
    else:
        mc = load_mcore(a.load_ckpt_path, num_layers=L, custom_layers=a.custom_pipeline_layers)
    if a.load_lora_ckpt_path:
        merge_lora_into(mc, torch.load(a.load_lora_ckpt_path, map_location="cpu"), a.lora_alpha, a.lora_dim)
    if dt is not None:
        mc = {k: (v.to(dt) if v.is_floating_point() else v) for k, v in mc.items()}
    if a.save_platform == "mcore":
        dump = {"tensor_model_parallel_size": a.tensor_model_parallel_size,
                "pipeline_model_parallel_size": a.pipeline_model_parallel_size,
                "expert_parallel_size": a.expert_parallel_size, "custom_pipeline_layers": a.custom_pipeline_layers,
                "num_layers": L, "num_attention_heads": H, "num_query_groups": G, "vocab_size": V, "num_experts": E}
        save_mcore(mc, a.save_ckpt_path, tp=a.tensor_model_parallel_size, pp=a.pipeline_model_parallel_size,
                   ep=a.expert_parallel_size, num_layers=L, num_experts=E, custom_layers=a.custom_pipeline_layers,
                   args_dump=dump)
    else:
        if composite:
            n_vit = 1 + max(int(k.split("image_encoder.decoder.layers.")[1].split(".")[0]) for k in mc
                            if "image_encoder.decoder.layers." in k)
            hf_out = nm.composite_vlm_mcore_to_hf(mc, fam, composite, vit_layers=a.vit_num_layers or n_vit, vit_heads=a.vit_num_heads,
                                                  num_layers=L, num_heads=H, num_groups=G, vocab_size=V, num_experts=E,
                                                  tie_embeddings=tie)
        elif vlm:
            n_vit = 1 + max(int(k.split("image_encoder.decoder.layers.")[1].split(".")[0]) for k in mc
                            if "image_encoder.decoder.layers." in k)
            hf_out = nm.vlm_mcore_to_hf(mc, fam, vit_layers=a.vit_num_layers or n_vit, vit_heads=a.vit_num_heads,
                                        num_layers=L, num_heads=H, num_groups=G, vocab_size=V, num_experts=E,
                                        tie_embeddings=tie)
        else:
            hf_out = nm.mcore_to_hf(mc, fam, num_layers=L, num_heads=H, num_groups=G, vocab_size=V, num_experts=E,
                                    tie_embeddings=tie)
        save_hf(hf_out, a.save_ckpt_path, hf_cfg or None)
    print(f"converted {len(mc)} tensors: {a.load_platform} -> {a.save_platform} at {a.save_ckpt_path}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
