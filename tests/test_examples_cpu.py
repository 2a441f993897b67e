"""Every launch script under examples/ must be valid shell and carry a flag set that the argument parser, the config
builder and the validators accept for the world size the script asks for."""
import glob
import os
import re
import shlex
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = sorted(glob.glob(os.path.join(ROOT, "examples", "**", "*.sh"), recursive=True))


def _train_args(text: str):
    """The arguments after ``-m loongforge_b200.train`` with shell variables replaced by plain values."""
    m = re.search(r"-m loongforge_b200\.train\s*\\?\n(.*)", text, re.S)
    if not m:
        return None
    body = m.group(1).replace("\\\n", " ")
    body = body.split("\n")[0] if "\n" in body.strip() and not body.strip().startswith("--") else body
    body = re.sub(r'"\$\{DATA_ARGS\[@\]\}"', "--mock-data", body)
    defaults = dict(re.findall(r"^([A-Z_]+)=\$\{\1:-([^}$]*)\}", text, re.M))  # VAR=${VAR:-default} lines
    defaults["GPUS"] = "8"
    _train_args.nnodes = int(defaults.get("NNODES", "1") or 1)
    body = re.sub(r'"?\$\{?([A-Z_]+)(:-[^}]*)?\}?"?', lambda m: defaults.get(m.group(1)) or "/tmp/x", body)
    return [a for a in shlex.split(body.strip().splitlines()[0] if "\n" in body else body) if a]


@pytest.mark.parametrize("path", SCRIPTS, ids=[os.path.relpath(p, ROOT) for p in SCRIPTS])
def test_example_script(path, monkeypatch):
    assert subprocess.run(["bash", "-n", path]).returncode == 0
    args = _train_args(open(path).read())
    if args is None:
        return  # tools / other entry points
    from loongforge_b200.config.arguments import parse_args
    from loongforge_b200.config.build import build_configs

    world = 8 * _train_args.nnodes                      # multi-node scripts carry NNODES=${NNODES:-n}
    monkeypatch.setenv("WORLD_SIZE", str(world))
    a, ov = parse_args(args)
    cfg, tc, dims, _ = build_configs(a, ov)
    assert tc.train_iters > 0 and world % (dims.tp * dims.pp * dims.cp) == 0
    stage = world // dims.pp
    assert stage % (dims.ep * dims.etp) == 0            # the expert mesh tiles the ranks of a pipeline stage


def test_launcher_planner_layouts():
    from loongforge_b200.models.registry import get_model_config
    from tools.generate_launchers import family_of, generate, plan, presets, stage_layers

    small = plan("llama3-8b")
    assert (small.tp, small.pp, small.nodes, small.recompute) == (1, 1, 1, "none") and small.est_gb < 126
    big = plan("llama3.1-405b")
    assert big.nodes > 1 and big.tp == 8 and big.pp > 1 and big.est_gb <= 126
    moe = plan("qwen3-235b-a22b")
    cfg = get_model_config("qwen3-235b-a22b")
    assert cfg.num_query_groups % moe.tp == 0 and moe.ep >= 8 and (moe.world // moe.pp) % moe.ep == 0
    assert sum(stage_layers(94, 4)) == 94 and stage_layers(94, 4) == [24, 24, 23, 23] and stage_layers(61, 2) == [31, 30]
    assert plan("qwen3-8b", "sft").seq_length == 8192
    assert family_of("qwen3-next-80b-a3b")[0] == "qwen3_next" and family_of("llama3.1-8b")[1] == "llama3"
    files = generate(write=False)
    on_disk = {os.path.relpath(p, ROOT) for p in SCRIPTS}
    assert set(files) <= on_disk, sorted(set(files) - on_disk)[:5]           # the committed scripts are the generator's output
    for rel in ("examples/qwen3/pretrain/pretrain_qwen3_8b.sh", "examples/llama3/finetuning/sft_llama3_8b_lora.sh"):
        assert open(os.path.join(ROOT, rel)).read() == files[rel]
    assert len(presets()) >= 55


EMBODIED = [p for p in SCRIPTS if "-m loongforge_b200.embodied.train" in open(p).read()]


@pytest.mark.parametrize("path", EMBODIED, ids=[os.path.relpath(p, ROOT) for p in EMBODIED])
def test_embodied_script_overrides_parse(path, monkeypatch):
    """The recipe and the key=value overrides of every embodied launcher are accepted by the embodied argument parser."""
    from loongforge_b200.embodied.config import parse_args

    text = open(path).read()
    m = re.search(r"-m loongforge_b200\.embodied\.train(.*)", text, re.S)
    body = m.group(1).replace("\\\n", " ")
    body = re.sub(r'"\$\{DATA_ARGS\[@\]\}"', "dataset_type=synthetic", body)
    body = re.sub(r"\$\{[A-Z]+:\+[^}]*\}", "", body)                      # ${VAR:+...}: absent by default
    body = body.replace('"$@"', "")
    body = re.sub(r'"?\$\{?OUT[^"\s]*"?', "/tmp/x", body)
    body = re.sub(r'"?\$\{?[A-Z_]+(:-[^}]*)?\}?"?', "/tmp/x", body)
    monkeypatch.chdir(ROOT)
    a = parse_args(shlex.split(body))
    assert a.model_name in path and a.train_steps > 0
    if "lora" in os.path.basename(path):
        assert a.lora_rank > 0 and a.lora_targets == []


def test_packaging_entry_points_resolve():
    import importlib
    import tomllib

    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as f:
        meta = tomllib.load(f)
    scripts = meta["project"]["scripts"]
    assert scripts["LoongForge"] == "loongforge.train:main"               # the reference's console script
    for target in scripts.values():
        mod, fn = target.split(":")
        assert callable(getattr(importlib.import_module(mod), fn)), target
