"""Plans a parallel layout for a model preset on B200 nodes and writes the launch scripts under ``examples/``.

    python -m tools.generate_launchers --list                       # the plan of every preset, as a table
    python -m tools.generate_launchers --model qwen3-32b --phase sft --stdout
    python -m tools.generate_launchers --write                      # (re)generate examples/<family>/{pretrain,finetuning,checkpoint_convert}/

The plan is a memory estimate against 180 GB per GPU, not a search: weights (bf16) + main gradients (fp32) stay on every
model-parallel rank, the optimizer state (fp32 master + two moments) is spread over the data-parallel ranks by the
distributed optimizer. Expert weights are divided by the expert-parallel size first (all GPUs of a node), the dense part
by tensor parallelism (2, 4, 8 inside a node, with sequence parallelism), then pipeline stages are added (whole layers
per stage, over nodes) until the estimate fits in 70 % of the memory; what is left of the 70 % decides between selective
and full recomputation. Scripts name the nodes through ``NNODES`` / ``NODE_RANK`` / ``MASTER_ADDR`` so that one file
serves every node of a job (the layout of the reference's examples/<family>/{pretrain,finetuning,checkpoint_convert}).
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import re
import sys
from typing import Dict, List, Optional, Tuple

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GPU_GB, BUDGET, GPUS_PER_NODE = 180.0, 0.70, 8

# preset prefix -> (examples directory, converter family, chat template)
FAMILY_OF = [
    ("deepseek-v2", ("deepseek_v2", "deepseek", "deepseek")), ("deepseek-v3", ("deepseek_v3", "deepseek", "deepseek")),
    ("deepseek-v4", ("deepseek_v4", None, "deepseek")), ("ernie4.5", ("ernie4.5", None, "chatml")),
    ("glm5.2", ("glm5.2", "glm", "chatml")), ("glm5", ("glm5", "glm", "chatml")), ("kimi-k2", ("kimi_k2.x", "kimi_k2", "chatml")),
    ("minicpm-v", ("minicpm_v_4_6", None, "chatml")), ("qwen3.6", ("qwen3.6", "qwen3_5", "chatml")), ("internlm2.5", ("internlm", "internlm2.5", "internlm2")),
    ("llama2", ("llama2", "llama2", "llama2")), ("llama3.1", ("llama3.1", "llama3", "llama3")),
    ("llama3", ("llama3", "llama3", "llama3")), ("mimo", ("mimo", "mimo", "chatml")),
    ("minimax", ("minimax", "minimax", "chatml")), ("qwen-", ("qwen", "qwen2", "chatml")),
    ("qwen1.5", ("qwen1.5", "qwen2", "chatml")), ("qwen2.5", ("qwen2.5", "qwen2.5", "chatml")),
    ("qwen2-", ("qwen2", "qwen2", "chatml")), ("qwen3-next", ("qwen3_next", "qwen3_next", "chatml")),
    ("qwen3.5", ("qwen3.5", "qwen3_5", "chatml")), ("qwen3", ("qwen3", "qwen3", "chatml")),
]


def family_of(name: str) -> Tuple[str, Optional[str], str]:
    for prefix, fam in FAMILY_OF:
        if name.startswith(prefix):
            return fam
    return (re.split(r"[-.]", name)[0], None, "chatml")


@dataclasses.dataclass
class Plan:
    model: str
    params_b: float
    tp: int = 1
    pp: int = 1
    ep: int = 1
    nodes: int = 1
    recompute: str = "none"        # none | selective | full
    seq_length: int = 4096
    micro_batch: int = 1
    est_gb: float = 0.0
    moe: bool = False
    uneven: bool = False
    num_layers: int = 0

    @property
    def world(self) -> int:
        return self.nodes * GPUS_PER_NODE

    def label(self) -> str:
        parts = [f"TP{self.tp}" + (" + SP" if self.tp > 1 else "")] if self.tp > 1 else []
        if self.pp > 1:
            parts.append(f"PP{self.pp}")
        if self.ep > 1:
            parts.append(f"EP{self.ep}")
        parts.append(f"DP{self.world // (self.tp * self.pp)}")
        return ", ".join(parts) + (f", {self.recompute} recompute" if self.recompute != "none" else "")


def _split_params(cfg) -> Tuple[float, float]:
    """(dense parameters, routed-expert parameters)."""
    total = cfg.num_parameters()
    if not cfg.num_moe_experts:
        return float(total), 0.0
    glu = 3 if cfg.gated_linear_unit else 2
    moe_layers = sum(cfg.is_moe_layer(i) for i in range(cfg.num_layers))
    experts = moe_layers * cfg.num_moe_experts * glu * cfg.hidden_size * cfg.moe_ffn_hidden_size
    return float(total - experts), float(experts)


def _estimate(cfg, tp, pp, ep, world, seq, recompute) -> float:
    dense, experts = _split_params(cfg)
    dp = max(world // (tp * pp), 1)
    edp = max(world // (ep * pp), 1)
    state = (dense / (tp * pp)) * (6 + 12 / dp) + (experts / (ep * pp)) * (6 + 12 / edp)
    layers = -(-cfg.num_layers // pp)
    per_layer = {"none": 34, "selective": 18, "full": 2}[recompute] * seq * cfg.hidden_size / tp   # bytes, one micro-batch
    act = layers * per_layer * min(pp, 4)                      # 1F1B keeps up to pp micro-batches in flight on stage 0
    logits = 0 if pp > 1 else 6 * seq * cfg.padded_vocab_size / tp
    return (state + act + logits) / 2 ** 30


def plan(model: str, phase: str = "pretrain", seq: Optional[int] = None) -> Plan:
    from loongforge_b200.models.registry import get_model_config
    cfg = get_model_config(model)
    seq = seq or (8192 if phase == "sft" else 4096)
    seq = min(seq, cfg.max_position_embeddings or seq)
    p = Plan(model, cfg.num_parameters() / 1e9, seq_length=seq, moe=bool(cfg.num_moe_experts))
    heads, groups = cfg.num_attention_heads, cfg.num_query_groups or cfg.num_attention_heads
    tps = [t for t in (1, 2, 4, 8) if heads % t == 0 and groups % t == 0]
    for nodes in (1, 2, 4, 8, 16, 32, 64):
        world = nodes * GPUS_PER_NODE
        for rc in ("none", "selective", "full"):
            for pp in (q for q in (1, 2, 4, 8, 16) if q <= cfg.num_layers and (q == 1 or q <= 2 * nodes)):
                for tp in tps:
                    if tp * pp > world:
                        continue
                    eps = [1]
                    if p.moe:  # experts over the GPUs of a node first, over more nodes only when that does not fit
                        eps = [e for e in (8, 16, 32, 64) if cfg.num_moe_experts % e == 0 and (world // pp) % e == 0] or \
                              [e for e in (4, 2, 1) if cfg.num_moe_experts % e == 0 and (world // pp) % e == 0][:1]
                    for ep in eps:
                        est = _estimate(cfg, tp, pp, ep, world, seq, rc)
                        if est <= GPU_GB * BUDGET:
                            p.tp, p.pp, p.ep, p.nodes, p.recompute, p.est_gb = tp, pp, ep, nodes, rc, est
                            p.uneven = cfg.num_layers % pp != 0
                            p.num_layers = cfg.num_layers
                            return p
    raise RuntimeError(f"no layout found for {model}")


def stage_layers(num_layers: int, pp: int) -> List[int]:
    """Layers per stage when they do not divide: the last stage (which also holds the output layer and the loss) gets
    the fewest, the first ones the extra layers."""
    base, extra = divmod(num_layers, pp)
    counts = [base + 1] * extra + [base] * (pp - extra)
    return counts


HEADER = """#!/bin/bash
# {title}
# Layout for {nodes} node(s) of 8 B200 ({label}); estimated {est:.0f} GB of 180 GB per GPU. Written by
# tools/generate_launchers.py; run it on every node with NODE_RANK set (one node: no variables needed).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
GPUS=${{GPUS:-8}}
NNODES=${{NNODES:-{nodes}}}
NODE_RANK=${{NODE_RANK:-0}}
MASTER_ADDR=${{MASTER_ADDR:-127.0.0.1}}
MASTER_PORT=${{MASTER_PORT:-29500}}
CKPT=${{CKPT:-$REPO/outputs/{slug}}}
"""


def _parallel_flags(p: Plan) -> List[str]:
    out = []
    if p.tp > 1:
        out.append(f"--tensor-model-parallel-size {p.tp} --sequence-parallel")
    if p.pp > 1:
        out.append(f"--pipeline-model-parallel-size {p.pp}"
                   + (f" --custom-pipeline-layers {','.join(map(str, stage_layers(p.num_layers, p.pp)))}" if p.uneven else ""))
    if p.ep > 1:
        out.append(f"--expert-model-parallel-size {p.ep} --moe-token-dispatcher-type alltoall --moe-grouped-gemm")
    out.append("--use-distributed-optimizer --overlap-grad-reduce --overlap-param-gather")
    if p.recompute == "selective":
        out.append("--recompute-granularity selective")
    elif p.recompute == "full":
        out.append("--recompute-granularity full --recompute-method uniform --recompute-num-layers 1")
    return out


def _launch(p: Plan, body: List[str]) -> str:
    lines = ['python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node "$GPUS" \\',
             '  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \\', "  -m loongforge_b200.train \\"]
    lines += [f"  {b} \\" for b in body[:-1]] + [f"  {body[-1]}"]
    return "\n".join(lines) + "\n"


def pretrain_script(p: Plan) -> str:
    slug = p.model.replace("-", "_").replace(".", "_")
    gbs = max(p.world // (p.tp * p.pp), 1) * 16
    head = HEADER.format(title=f"{p.model} ({p.params_b:.1f} B parameters) pretraining, sequence length {p.seq_length}", nodes=p.nodes,
                         label=p.label(), est=p.est_gb, slug=slug)
    head += ('DATA_PATH=${DATA_PATH:-}\nexport PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True\nDATA_ARGS=(--mock-data)\n'
             '[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH" --split 99,1,0)\n\ncd "$REPO"\n')
    body = [f"--model-name {p.model}"] + _parallel_flags(p) + [
        f"--micro-batch-size {p.micro_batch} --global-batch-size {gbs} --seq-length {p.seq_length}",
        "--bf16 --lr 3e-4 --min-lr 3e-5 --lr-decay-style cosine --lr-warmup-fraction 0.01 --weight-decay 0.1",
        "--adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0",
        "--train-iters 5000 --log-interval 10 --log-throughput",
        '--save "$CKPT" --save-interval 500 --ckpt-format torch_dist', '"${DATA_ARGS[@]}"']
    return head + _launch(p, body)


def sft_script(p: Plan, lora: bool = False) -> str:
    slug = "sft_" + p.model.replace("-", "_").replace(".", "_") + ("_lora" if lora else "")
    gbs = max(p.world // (p.tp * p.pp), 1) * 8
    head = HEADER.format(title=f"{p.model} chat fine-tuning{' with LoRA' if lora else ''}, packed sequences of {p.seq_length} tokens",
                         nodes=p.nodes, label=p.label(), est=p.est_gb, slug=slug)
    head += ('DATA_PATH=${DATA_PATH:-}\nTOKENIZER=${TOKENIZER:-}   # Hugging Face tokenizer directory\nLOAD=${LOAD:-}             # converted base checkpoint\n'
             'export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True\nDATA_ARGS=(--mock-data)\n'
             '[ -n "$DATA_PATH" ] && DATA_ARGS=(--sft-dataset "$DATA_PATH" --tokenizer-type HFTokenizer --hf-tokenizer-path "$TOKENIZER")\n'
             '[ -n "$LOAD" ] && DATA_ARGS+=(--load "$LOAD" --finetune)\n\ncd "$REPO"\n')
    body = [f"--model-name {p.model}"] + _parallel_flags(p) + [
        f"--micro-batch-size 1 --global-batch-size {gbs} --seq-length {p.seq_length}",
        f"--bf16 --lr {'1e-4' if lora else '1e-5'} --min-lr 1e-6 --lr-decay-style cosine --lr-warmup-fraction 0.01 --weight-decay 0.1",
        "--adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0",
        f"--training-phase sft --packing-sft-data --chat-template {family_of(p.model)[2]}"]
    if lora:
        body.append("--peft-type lora --lora-rank 16 --lora-alpha 32")
    body += ["--train-iters 1000 --log-interval 10 --log-throughput", '--save "$CKPT" --save-interval 500 --ckpt-format torch_dist',
             '"${DATA_ARGS[@]}"']
    return head + _launch(p, body)


def convert_script(p: Plan, direction: str, family: str) -> str:
    slug = p.model.replace("-", "_").replace(".", "_")
    fam = family + ("_moe" if family == "qwen3" and p.moe else "")
    par = f"--tensor_model_parallel_size {p.tp} --pipeline_model_parallel_size {p.pp}" + (f" --expert_parallel_size {p.ep}" if p.ep > 1 else "")
    if direction == "hf_to_mcore":
        return (f"#!/bin/bash\n# Hugging Face {p.model} checkpoint -> training layout sharded for {p.label().split(', DP')[0] or 'one GPU'}.\n"
                "set -euo pipefail\nREPO=$(cd \"$(dirname \"$0\")/../../..\" && pwd)\n"
                "HF=${1:?path to the Hugging Face checkpoint directory}\n"
                f"OUT=${{2:-$REPO/outputs/{slug}_mcore}}\ncd \"$REPO\"\n"
                "python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \\\n"
                f"  --model_type_custom {fam} --load_ckpt_path \"$HF\" --save_ckpt_path \"$OUT\" \\\n"
                f"  {par} --safetensors --torch_dtype bfloat16\n")
    return (f"#!/bin/bash\n# Training checkpoint of {p.model} -> Hugging Face safetensors (shards of any TP / PP / EP layout are merged).\n"
            "set -euo pipefail\nREPO=$(cd \"$(dirname \"$0\")/../../..\" && pwd)\n"
            "IN=${1:?path to the training checkpoint}\n"
            f"OUT=${{2:-$REPO/outputs/{slug}_hf}}\ncd \"$REPO\"\n"
            "python -m tools.convert_checkpoint.convert --load_platform mcore --save_platform huggingface \\\n"
            f"  --model_type_custom {fam} --load_ckpt_path \"$IN\" --save_ckpt_path \"$OUT\" --safetensors --torch_dtype bfloat16\n")


# VLM name (first line of its YAML) -> (examples directory, language-model preset)
def vlm_presets() -> Dict[str, Tuple[str, str]]:
    """Vision-language models registered by the YAML files under configs/models, with the language preset they compose."""
    import yaml as _yaml
    from loongforge_b200.config import build as B
    from loongforge_b200.models.registry import list_models
    llms = {m.replace("-", "_").replace(".", "_"): m for m in list_models()}
    dirs = {"qwen2.5vl": "qwen2.5_vl", "qwen3vl": "qwen3_vl", "internvl": "internvl", "llavaov": "llava_onevision_1.5",
            "ernie4.5vl": "ernie4.5", "kimi_k2": "kimi_k2.x", "glm": "glm5.2_vit", "custom": "custom"}
    out: Dict[str, Tuple[str, str]] = {}
    for name, rel in sorted(B._scan_model_yaml().items()):
        with open(os.path.join(B.CONFIG_DIR, rel)) as f:
            node = _yaml.safe_load(f.read().replace("${", "$("))     # resolvers are not needed here
        if not isinstance(node, dict) or "defaults" not in node:
            continue
        llm = None
        for d in node["defaults"]:
            if isinstance(d, dict):
                for k, v in d.items():
                    if k.endswith("@model.foundation"):
                        llm = llms.get(str(v).replace("_llm", "")) or llms.get(str(v))
        if llm:
            out[name] = (dirs.get(rel.split("/")[0], rel.split("/")[0]), llm)
    return out


def vlm_sft_script(name: str, llm: str) -> str:
    p = plan(llm, "sft", 4096)
    slug = "sft_" + name.replace("-", "_").replace(".", "_")
    gbs = max(p.world // (p.tp * p.pp), 1) * 4
    head = HEADER.format(title=f"{name} supervised fine-tuning on image-text conversations (language model: {llm}); the vision encoder keeps\n"
                               f"# tensor-parallel size 1 and is spread over the TP ranks by encoder heterogeneous DP", nodes=p.nodes,
                         label=p.label(), est=p.est_gb, slug=slug)
    head += ('DATA_PATH=${DATA_PATH:-}        # WebDataset shards written by tools/data_preprocess/vlm_to_webdataset.py\n'
             'TOKENIZER=${TOKENIZER:-}\nexport PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True\nDATA_ARGS=(--mock-data)\n'
             '[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH" --tokenizer-type HFTokenizer --hf-tokenizer-path "$TOKENIZER")\n\ncd "$REPO"\n').replace("\\n", "\n")
    par = _parallel_flags(p)
    if p.tp > 1:
        par[0] += " --encoder-tensor-model-parallel-size 1"
    body = [f"--model-name {name} --training-phase sft"] + par + [
        f"--micro-batch-size 1 --global-batch-size {gbs} --seq-length 4096 --packing-sft-data --variable-seq-lengths",
        "--bf16 --lr 1e-5 --min-lr 1e-6 --lr-decay-style cosine --lr-warmup-fraction 0.03 --weight-decay 0.1 --clip-grad 1.0",
        "--train-iters 1000 --log-interval 5 --log-throughput", '--save "$CKPT" --save-interval 250 --ckpt-format torch_dist',
        '"${DATA_ARGS[@]}"', "+model.image_encoder.freeze=True"]
    return head + _launch(p, body)


EMBODIED = {  # policy -> (strategy, extra overrides, world model?)
    "pi05": ("ddp", "ddp_comm_hook=bf16_compress per_device_batch_size=16", False),
    "groot_n1_6": ("ddp", "per_device_batch_size=16", False),
    "groot_n1_7": ("ddp", "per_device_batch_size=16", False),
    "xvla": ("ddp", "per_device_batch_size=16", False),
    "lingbot_va": ("fsdp", "'fsdp_wrap_patterns=[auto]' fsdp_reduce_dtype=fp32 per_device_batch_size=2", True),
    "fastwam": ("zero1", "per_device_batch_size=2", True),
    "dreamzero": ("fsdp", "'fsdp_wrap_patterns=[auto]' fsdp_reduce_dtype=fp32 per_device_batch_size=1", True),
    "cosmos3": ("fsdp", "'fsdp_wrap_patterns=[auto]' fsdp_reduce_dtype=fp32 per_device_batch_size=2", True),
}

_EMB_HEAD = """#!/bin/bash
# {title}
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
GPUS=${{GPUS:-8}}
OUT=${{OUT:-$REPO/outputs/{slug}}}
DATA=${{DATA:-}}            # LeRobot v2 data set directory (empty: synthetic episodes)
DATA_ARGS=(dataset_type=synthetic)
[ -n "$DATA" ] && DATA_ARGS=(dataset_type=lerobot dataset_path="$DATA" use_transforms=true stats_path="$DATA")
cd "$REPO"
"""


def embodied_scripts() -> Dict[str, str]:
    out: Dict[str, str] = {}
    for name, (strategy, extra, world) in EMBODIED.items():
        run = ('python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \\\n'
               f"  -m loongforge_b200.embodied.train --config configs/embodied/{name}.yaml \\\n")
        cache = ' ${CACHE:+precomputed_cache="$CACHE"}' if world else ""
        out[f"examples/embodied/{name}/finetune_{name}.sh"] = (
            _EMB_HEAD.format(title=f"Fine-tune the {name} policy ({strategy}); key=value tokens after the script name override the recipe."
                             + ("\n# CACHE=<dir> trains from features written by precompute_" + name + ".sh." if world else ""), slug=name)
            + run + f"  strategy={strategy} {extra} train_steps=2000 save_interval=500 log_stage_times=true \\\n"
            + f'  output_dir="$OUT" "${{DATA_ARGS[@]}}"{cache} "$@"\n')
        out[f"examples/embodied/{name}/finetune_{name}_lora.sh"] = (
            _EMB_HEAD.format(title=f"LoRA fine-tuning of {name}: adapters on the policy's default projections, base weights from PRETRAINED.", slug=name + "_lora")
            + 'PRETRAINED=${PRETRAINED:-}\n' + run
            + "  strategy=ddp lora_rank=16 lora_alpha=32 'lora_targets=[]' per_device_batch_size=4 lr=2e-4 train_steps=2000 save_interval=500 \\\n"
            + '  output_dir="$OUT" "${DATA_ARGS[@]}" ${PRETRAINED:+pretrained_checkpoint="$PRETRAINED"} "$@"\n')
        out[f"examples/embodied/{name}/eval_{name}.sh"] = (
            f"#!/bin/bash\n# Serve the newest checkpoint of a {name} run and roll out evaluation episodes against it.\nset -euo pipefail\n"
            'REPO=$(cd "$(dirname "$0")/../../.." && pwd)\nRUN=${1:?run directory (output_dir of the training)}\nPORT=${PORT:-18600}\ncd "$REPO"\n'
            f'python -m loongforge_b200.embodied.eval serve --checkpoint "$RUN" --port "$PORT" model_name={name} output_dir="$RUN" &\n'
            'SERVER=$!\ntrap \'kill "$SERVER"\' EXIT\nsleep 20\n'
            'python -m loongforge_b200.embodied.eval run --port "$PORT" --episodes "${EPISODES:-20}" --output-dir "$RUN/eval"\n')
        if world:
            out[f"examples/embodied/{name}/precompute_{name}.sh"] = (
                f"#!/bin/bash\n# Cache the codec latents / text embeddings of a data set for {name} (train afterwards with CACHE=<dir>).\nset -euo pipefail\n"
                'REPO=$(cd "$(dirname "$0")/../../.." && pwd)\nDATA=${1:?LeRobot v2 data set directory}\nCACHE=${2:?output directory}\ncd "$REPO"\n'
                f'python -m tools.data_preprocess.embodied_precompute build --output "$CACHE" --config configs/embodied/{name}.yaml \\\n'
                '  dataset_type=lerobot dataset_path="$DATA" ${PRETRAINED:+pretrained_checkpoint="$PRETRAINED"}\n'
                f'python -m tools.data_preprocess.embodied_precompute validate --cache "$CACHE" --deep\n')
    return out


def presets() -> List[str]:
    from loongforge_b200.models.registry import list_models
    skip = ("tiny-", "qwen2.5-vit", "minicpm-v-4.6-llm")
    return [m for m in list_models() if not m.startswith(skip) and not m.endswith(("-slice", "-warmup", "-sparse"))]


def generate(write: bool) -> Dict[str, str]:
    files: Dict[str, str] = {}
    for m in presets():
        d, conv, _ = family_of(m)
        slug = m.replace("-", "_").replace(".", "_")
        pp = plan(m, "pretrain")
        files[f"examples/{d}/pretrain/pretrain_{slug}.sh"] = pretrain_script(pp)
        ps = plan(m, "sft")
        files[f"examples/{d}/finetuning/sft_{slug}.sh"] = sft_script(ps)
        if ps.params_b < 40 and not ps.moe:
            files[f"examples/{d}/finetuning/sft_{slug}_lora.sh"] = sft_script(ps, lora=True)
        if conv:
            files[f"examples/{d}/checkpoint_convert/convert_{slug}_hf_to_mcore.sh"] = convert_script(pp, "hf_to_mcore", conv)
            files[f"examples/{d}/checkpoint_convert/convert_{slug}_mcore_to_hf.sh"] = convert_script(pp, "mcore_to_hf", conv)
    for name, (d, llm) in vlm_presets().items():
        files[f"examples/{d}/finetuning/sft_{name.replace('-', '_').replace('.', '_')}.sh"] = vlm_sft_script(name, llm)
    files.update(embodied_scripts())
    if write:
        for rel, text in files.items():
            path = os.path.join(ROOT, rel)
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w") as f:
                f.write(text)
            os.chmod(path, 0o755)
    return files


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--write", action="store_true")
    ap.add_argument("--model", default=None)
    ap.add_argument("--phase", default="pretrain", choices=["pretrain", "sft", "sft_lora"])
    ap.add_argument("--seq-length", type=int, default=None)
    ap.add_argument("--stdout", action="store_true")
    a = ap.parse_args(argv)
    if a.list:
        print(f"{'model':28s} {'B params':>9s} {'nodes':>5s}  layout (pretrain)")
        for m in presets():
            p = plan(m)
            print(f"{m:28s} {p.params_b:9.1f} {p.nodes:5d}  {p.label()}  ~{p.est_gb:.0f} GB")
    if a.model:
        p = plan(a.model, "sft" if a.phase.startswith("sft") else "pretrain", a.seq_length)
        text = pretrain_script(p) if a.phase == "pretrain" else sft_script(p, lora=a.phase == "sft_lora")
        if a.stdout or not a.write:
            print(text)
    if a.write and not a.model:
        files = generate(True)
        print(f"wrote {len(files)} launch scripts")
    return 0


if __name__ == "__main__":
    sys.exit(main())
