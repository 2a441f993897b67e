"""Episode records and reports of the evaluation framework.

* ``results.jsonl``: one record per finished episode (suite, task, task id, episode, seed, success, steps, failure reason,
  latencies); appended as episodes finish, so an interrupted evaluation resumes where it stopped (``completed_keys``);
* summaries per task and per suite: success rate, binomial standard error, Wilson 95 % interval, mean steps, failure
  reasons by count; CSV files of both; a floor check (every task has at least ``min_episodes`` episodes);
* ``write_report``: ``report.json`` + ``report.md`` with the summaries, latency percentiles, the failures, and what is needed
  to reproduce the run (arguments, host resources, read-only GPU query, source revision).

(reference: loongforge/embodied/eval/metrics/results.py:18-245, metrics/report.py:23-401)
"""
from __future__ import annotations

import collections
import csv
import json
import math
import os
import subprocess
import time
from typing import Any, Dict, Iterable, List, Optional, Set, Tuple

Record = Dict[str, Any]
Key = Tuple[str, str, int, int]


def append_jsonl(path: str, record: Record) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "a") as f:
        f.write(json.dumps(record) + "\n")


def load_jsonl(path: str) -> List[Record]:
    if not os.path.isfile(path):
        return []
    out = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                try:
                    out.append(json.loads(line))
                except json.JSONDecodeError:  # a line cut off by an interruption: the episode runs again
                    continue
    return out


def episode_key(r: Record) -> Key:
    return (str(r.get("suite", "")), str(r.get("task", "")), int(r.get("episode", 0)), int(r.get("seed", 0)))


def completed_keys(records: Iterable[Record]) -> Set[Key]:
    return {episode_key(r) for r in records if "success" in r}


def wilson_interval(successes: int, n: int, z: float = 1.96) -> Tuple[float, float]:
    if n == 0:
        return 0.0, 1.0
    p = successes / n
    den = 1 + z * z / n
    centre = (p + z * z / (2 * n)) / den
    half = z * math.sqrt(p * (1 - p) / n + z * z / (4 * n * n)) / den
    return max(0.0, centre - half), min(1.0, centre + half)


def _summary(records: List[Record]) -> Dict[str, Any]:
    n = len(records)
    k = sum(bool(r["success"]) for r in records)
    rate = k / n if n else 0.0
    lo, hi = wilson_interval(k, n)
    reasons = collections.Counter(str(r.get("failure_reason") or "unknown") for r in records if not r["success"])
    steps = [r["steps"] for r in records if "steps" in r]
    return {"episodes": n, "successes": k, "success_rate": rate, "stderr": math.sqrt(rate * (1 - rate) / n) if n else 0.0,
            "ci95": [lo, hi], "mean_steps": sum(steps) / len(steps) if steps else None,
            "failure_reasons": dict(reasons.most_common())}


def summarize_tasks(records: Iterable[Record]) -> List[Dict[str, Any]]:
    groups: Dict[Tuple[str, str], List[Record]] = collections.defaultdict(list)
    for r in records:
        if "success" in r:
            groups[(str(r.get("suite", "")), str(r.get("task", "")))].append(r)
    return [{"suite": s, "task": t, **_summary(rs)} for (s, t), rs in sorted(groups.items())]


def summarize_suites(records: Iterable[Record], min_episodes: int = 1) -> List[Dict[str, Any]]:
    """Per suite over all its episodes, plus the mean of the per-task rates (tasks with fewer than ``min_episodes``
    episodes are listed as short and left out of that mean)."""
    records = [r for r in records if "success" in r]
    out = []
    for suite in sorted({str(r.get("suite", "")) for r in records}):
        rs = [r for r in records if str(r.get("suite", "")) == suite]
        tasks = [t for t in summarize_tasks(rs)]
        full = [t for t in tasks if t["episodes"] >= min_episodes]
        out.append({"suite": suite, **_summary(rs), "tasks": len(tasks),
                    "task_mean_success_rate": sum(t["success_rate"] for t in full) / len(full) if full else None,
                    "short_tasks": [t["task"] for t in tasks if t["episodes"] < min_episodes]})
    return out


def validate_episode_floor(records: Iterable[Record], min_episodes: int) -> List[Dict[str, Any]]:
    return [{"suite": t["suite"], "task": t["task"], "episodes": t["episodes"], "required": min_episodes}
            for t in summarize_tasks(records) if t["episodes"] < min_episodes]


def write_csv(path: str, rows: List[Dict[str, Any]]) -> None:
    if not rows:
        return
    cols = [c for c in rows[0] if not isinstance(rows[0][c], (dict, list))] + ["ci95_low", "ci95_high"]
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=cols, extrasaction="ignore")
        w.writeheader()
        for r in rows:
            w.writerow({**r, "ci95_low": r["ci95"][0], "ci95_high": r["ci95"][1]})


def latency_summary(records: Iterable[Record]) -> Dict[str, float]:
    vals = sorted(v for r in records for v in r.get("round_trip_ms", []))
    if not vals:
        return {}
    pick = lambda q: vals[min(len(vals) - 1, int(q * (len(vals) - 1) + 0.5))]  # noqa: E731
    server = [v for r in records for v in r.get("server_ms", []) if v is not None]
    return {"calls": len(vals), "mean": sum(vals) / len(vals), "p50": pick(0.5), "p95": pick(0.95), "p99": pick(0.99),
            "max": vals[-1], "server_mean": sum(server) / len(server) if server else None}


def resource_snapshot() -> Dict[str, Any]:
    """Host load, memory, disk, and a read-only GPU query (nothing is changed on the device)."""
    import psutil
    snap: Dict[str, Any] = {"time": time.strftime("%Y-%m-%d %H:%M:%S"), "cpu_count": psutil.cpu_count(),
                            "loadavg": list(os.getloadavg()) if hasattr(os, "getloadavg") else None,
                            "memory_total_gb": psutil.virtual_memory().total / 2 ** 30,
                            "memory_available_gb": psutil.virtual_memory().available / 2 ** 30,
                            "disk_free_gb": psutil.disk_usage(os.getcwd()).free / 2 ** 30}
    try:
        q = subprocess.run(["nvidia-smi", "--query-gpu=index,name,memory.used,memory.total,utilization.gpu", "--format=csv,noheader"],
                           capture_output=True, text=True, timeout=10)
        snap["gpus"] = q.stdout.strip().splitlines() if q.returncode == 0 else None
    except (OSError, subprocess.TimeoutExpired):
        snap["gpus"] = None
    return snap


def source_revision(repo: Optional[str] = None) -> Dict[str, Optional[str]]:
    repo = repo or os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

    def git(*a):
        try:
            r = subprocess.run(["git", "-C", repo, *a], capture_output=True, text=True, timeout=10)
            return r.stdout.strip() if r.returncode == 0 else None
        except (OSError, subprocess.TimeoutExpired):
            return None
    return {"commit": git("rev-parse", "HEAD"), "dirty": (git("status", "--porcelain") or "") != ""}


def _f(v) -> str:
    return "-" if v is None else f"{v:.3f}" if isinstance(v, float) else str(v)


def render_markdown(report: Dict[str, Any]) -> str:
    L = [f"# Evaluation report: {report.get('name', 'run')}", "",
         f"Policy: `{json.dumps(report.get('policy', {}))}`", ""]
    L += ["## Suites", "", "| suite | episodes | success rate | 95 % interval | task mean | mean steps |", "|---|---|---|---|---|---|"]
    for s in report["suites"]:
        L.append(f"| {s['suite']} | {s['episodes']} | {_f(s['success_rate'])} ± {_f(s['stderr'])} | "
                 f"[{_f(s['ci95'][0])}, {_f(s['ci95'][1])}] | {_f(s['task_mean_success_rate'])} | {_f(s['mean_steps'])} |")
    L += ["", "## Tasks", "", "| suite | task | episodes | successes | success rate | 95 % interval | failures |", "|---|---|---|---|---|---|---|"]
    for t in report["tasks"]:
        fails = ", ".join(f"{k}: {v}" for k, v in t["failure_reasons"].items()) or "-"
        L.append(f"| {t['suite']} | {t['task']} | {t['episodes']} | {t['successes']} | {_f(t['success_rate'])} | "
                 f"[{_f(t['ci95'][0])}, {_f(t['ci95'][1])}] | {fails} |")
    if report.get("floor_violations"):
        L += ["", "## Tasks below the episode floor", ""] + [f"* {v['suite']} / {v['task']}: {v['episodes']} of {v['required']}"
                                                            for v in report["floor_violations"]]
    lat = report.get("latency_ms") or {}
    if lat:
        L += ["", "## Latency (ms)", "", "| calls | mean | p50 | p95 | p99 | max | server mean |", "|---|---|---|---|---|---|---|",
              "| " + " | ".join(_f(lat.get(k)) for k in ("calls", "mean", "p50", "p95", "p99", "max", "server_mean")) + " |"]
    if report.get("failures"):
        L += ["", "## Failed episodes", ""] + [f"* {f['suite']} / {f['task']} episode {f['episode']} (seed {f['seed']}): "
                                               f"{f.get('failure_reason') or 'unknown'} after {f.get('steps', '?')} steps"
                                               for f in report["failures"][:50]]
    L += ["", "## Reproduction", "", "```json", json.dumps(report.get("reproduction", {}), indent=1), "```", ""]
    return "\n".join(L)


def write_report(output_dir: str, records: List[Record], *, name: str = "run", policy: Optional[dict] = None,
                 config: Optional[dict] = None, min_episodes: int = 1, resources: Optional[dict] = None) -> Dict[str, Any]:
    tasks, suites = summarize_tasks(records), summarize_suites(records, min_episodes)
    done = [r for r in records if "success" in r]
    report = {"name": name, "policy": policy or {}, "suites": suites, "tasks": tasks,
              "success_rate": sum(bool(r["success"]) for r in done) / len(done) if done else 0.0,
              "mean_steps": sum(r.get("steps", 0) for r in done) / len(done) if done else 0.0,
              "floor_violations": validate_episode_floor(records, min_episodes), "latency_ms": latency_summary(done),
              "failures": [{k: r.get(k) for k in ("suite", "task", "episode", "seed", "steps", "failure_reason")}
                           for r in done if not r["success"]],
              "episodes": [{k: r.get(k) for k in ("suite", "task", "episode", "seed", "success", "steps")} for r in done],
              "resources": resources or {},
              "reproduction": {"config": config or {}, "host": resource_snapshot(), "source": source_revision()}}
    os.makedirs(output_dir, exist_ok=True)
    with open(os.path.join(output_dir, "report.json"), "w") as f:
        json.dump(report, f, indent=1)
    with open(os.path.join(output_dir, "report.md"), "w") as f:
        f.write(render_markdown(report))
    write_csv(os.path.join(output_dir, "summary_tasks.csv"), tasks)
    write_csv(os.path.join(output_dir, "summary_suites.csv"), suites)
    return report
