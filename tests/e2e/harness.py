"""End-to-end regression harness: a YAML scenario names a training command; the harness runs it, parses the log line
of every iteration, and compares loss and gradient norm (2 % relative) and, when requested, time / throughput /
memory (5 % relative) with a recorded JSON baseline — the scheme of the reference's CI
(tests/llm_vlm/main.py:70-163, tasks/base_task.py:481-606, baselines tests/llm_vlm/baseline/**).

Scenario file::

    name: tiny_llama_pretrain
    nproc: 1                      # > 1 launches torchrun with the gloo backend
    args: [--model-name, tiny-llama, --train-iters, "6", ...]
    baseline: tiny_llama_pretrain.json
    check: [lm_loss, grad_norm]   # add elapsed_time_ms / throughput / mem_max_allocated_mb on fixed hardware
    skip_iterations: 1            # warm-up iterations excluded from timing checks

Run ``python -m tests.e2e.harness <scenario.yaml> [--update-baseline]``."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from typing import Dict, List, Optional

import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
TOLERANCE = {"lm_loss": 0.02, "grad_norm": 0.02, "elapsed_time_ms": 0.05, "throughput": 0.05, "mem_allocated_mb": 0.05,
             "mem_max_allocated_mb": 0.05}
TIMING_KEYS = ("elapsed_time_ms", "throughput")


def run_embodied_scenario(sc: dict, timeout: float = 900.0) -> List[dict]:
    """Embodied scenarios run ``loongforge_b200.embodied.train`` and are read back from its ``metrics.jsonl``
    (reference: tests/embodied/execution/metrics.py:6-24)."""
    import tempfile

    with tempfile.TemporaryDirectory() as out:
        cmd = [sys.executable, "-m", "loongforge_b200.embodied.train"] + [str(a) for a in sc["args"]] + [f"output_dir={out}"]
        env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", ""), PYTHONPATH=ROOT)
        p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
        if p.returncode != 0:
            raise RuntimeError(f"scenario {sc['name']} exited with {p.returncode}:\n{p.stdout[-2000:]}\n{p.stderr[-2000:]}")
        recs = []
        with open(os.path.join(out, "metrics.jsonl")) as f:
            for line in f:
                r = json.loads(line)
                recs.append({"iteration": r["step"], "lm_loss": r["loss"], "grad_norm": r["grad_norm"],
                             "elapsed_time_ms": r["elapsed_ms"], "throughput": r["samples_per_sec"]})
        return recs


def run_scenario_command(sc: dict, timeout: float = 900.0) -> List[dict]:
    if sc.get("stack") == "embodied":
        return run_embodied_scenario(sc, timeout)
    sys.path.insert(0, ROOT)
    from tools.log2json import parse

    nproc = int(sc.get("nproc", 1))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", ""), PYTHONPATH=ROOT)
    if nproc > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(sc.get("port", 29621)), "-m", "loongforge_b200.train",
               "--distributed-backend", "gloo"]
    else:
        cmd = [sys.executable, "-m", "loongforge_b200.train"]
    cmd += [str(a) for a in sc["args"]]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    if p.returncode != 0:
        raise RuntimeError(f"scenario {sc['name']} exited with {p.returncode}:\n{p.stdout[-2000:]}\n{p.stderr[-2000:]}")
    recs = parse(p.stdout.splitlines())
    if not recs:
        raise RuntimeError(f"scenario {sc['name']} printed no iteration lines")
    return recs


def compare(records: List[dict], baseline: List[dict], keys: List[str], skip_iterations: int = 1,
            tolerance: Optional[Dict[str, float]] = None) -> List[str]:
    tol = {**TOLERANCE, **(tolerance or {})}
    errors = []
    if len(records) != len(baseline):
        errors.append(f"{len(records)} iterations logged, baseline has {len(baseline)}")
    for r, b in zip(records, baseline):
        for k in keys:
            if k in TIMING_KEYS and r["iteration"] <= skip_iterations:
                continue
            if k not in r or k not in b:
                errors.append(f"iteration {r['iteration']}: {k} missing")
                continue
            rel = abs(r[k] - b[k]) / max(abs(b[k]), 1e-12)
            if rel > tol[k]:
                errors.append(f"iteration {r['iteration']}: {k} {r[k]:.6g} vs baseline {b[k]:.6g} ({rel:.1%} > {tol[k]:.0%})")
    return errors


def run(scenario_path: str, update_baseline: bool = False) -> List[str]:
    with open(scenario_path) as f:
        sc = yaml.safe_load(f)
    base_path = os.path.join(os.path.dirname(scenario_path), "..", "baseline", sc["baseline"])
    records = run_scenario_command(sc)
    if update_baseline or not os.path.isfile(base_path):
        os.makedirs(os.path.dirname(base_path), exist_ok=True)
        with open(base_path, "w") as f:
            json.dump(records, f, indent=1)
        return []
    with open(base_path) as f:
        baseline = json.load(f)
    return compare(records, baseline, sc.get("check", ["lm_loss", "grad_norm"]), sc.get("skip_iterations", 1),
                   sc.get("tolerance"))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("scenario")
    ap.add_argument("--update-baseline", action="store_true")
    a = ap.parse_args(argv)
    errs = run(a.scenario, a.update_baseline)
    for e in errs:
        print("MISMATCH", e)
    print("PASS" if not errs else f"FAIL ({len(errs)} mismatches)")
    return 1 if errs else 0


if __name__ == "__main__":
    sys.exit(main())
