"""Parse training stdout into per-iteration JSON records, with the same regular expressions the
reference's CI uses on its own log line (tests/llm_vlm/tools/log2json.py:19-29)."""
from __future__ import annotations

import json
import re
import sys

PATTERNS = {
    "iteration": r"iteration\s+(\d+)/\s*(\d+)",
    "elapsed_time_ms": r"elapsed time per iteration \(ms\):\s*([\d.]+)",
    "throughput": r"throughput \(token/sec/GPU\):\s*([\d.]+)",
    "tflops": r"flop throughput \(TFLOP/sec/GPU\):\s*([\d.]+)",
    "lm_loss": r"lm loss:\s*([\d.Ee+-]+)",
    "grad_norm": r"grad norm:\s*([\d.]+)",
    "mem_allocated_mb": r"mem-allocated-bytes-avg\(MB\):\s*([\d.]+)",
    "mem_max_allocated_mb": r"mem-max-allocated-bytes-avg\(MB\):\s*([\d.]+)",
}


def parse(lines):
    out = []
    for ln in lines:
        m = re.search(PATTERNS["iteration"], ln)
        if not m:
            continue
        rec = {"iteration": int(m.group(1)), "train_iters": int(m.group(2))}
        for k, pat in PATTERNS.items():
            if k == "iteration":
                continue
            mm = re.search(pat, ln)
            if mm:
                rec[k] = float(mm.group(1))
        out.append(rec)
    return out


if __name__ == "__main__":
    src = open(sys.argv[1]) if len(sys.argv) > 1 else sys.stdin
    json.dump(parse(src), sys.stdout, indent=1)
