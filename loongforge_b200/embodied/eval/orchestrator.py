"""Evaluation orchestrator: starts (or connects to) a policy server, rolls out episodes in environment adapters,
collects success / latency / resource metrics, writes a report and compares reports (reference:
loongforge/embodied/eval/orchestrator/*, adapters/*, metrics/*).

Environment adapters implement ``reset() -> Observation`` and ``step(action) -> (Observation, done, success)``. The
simulator adapters of the reference (LIBERO, CALVIN, SimplerEnv, RoboTwin, ManiSkill) render through a graphics stack
and are registered here as unavailable; ``ReachEnv`` is a headless kinematic task that exercises the whole loop."""
from __future__ import annotations

import dataclasses
import json
import os
import time
from typing import Callable, Dict, List, Optional

import numpy as np

from .protocol import ActionChunk, Observation
from .transport import RPCClient


class ReachEnv:
    """Headless point-reaching task: the state is (position, goal); actions are joint-space position targets; success
    when the position is within `tol` of the goal. Images are a rendered 2-D occupancy of position and goal."""

    def __init__(self, dim: int = 3, max_steps: int = 40, tol: float = 0.05, seed: int = 0, image_size: int = 32):
        self.dim, self.max_steps, self.tol, self.rng, self.S = dim, max_steps, tol, np.random.default_rng(seed), image_size
        self.episode = -1

    def _obs(self) -> Observation:
        img = np.zeros((self.S, self.S, 3), np.uint8)
        for ch, p in ((0, self.pos), (1, self.goal)):
            ij = np.clip(((p[:2] + 1) / 2 * (self.S - 1)).astype(int), 0, self.S - 1)
            img[ij[1], ij[0], ch] = 255
        return Observation({"front": img}, np.concatenate([self.pos, self.goal]).astype(np.float32),
                           "reach the green goal", self.episode, self.t)

    def reset(self) -> Observation:
        self.episode += 1
        self.t = 0
        self.pos = self.rng.uniform(-0.5, 0.5, self.dim)
        self.goal = self.rng.uniform(-0.5, 0.5, self.dim)
        return self._obs()

    def step(self, action: np.ndarray):
        self.pos = np.clip(action[:self.dim], -1, 1).astype(np.float64)
        self.t += 1
        success = bool(np.linalg.norm(self.pos - self.goal) < self.tol)
        return self._obs(), success or self.t >= self.max_steps, success


def _unavailable(name: str):
    def make(*a, **kw):
        raise RuntimeError(f"environment adapter {name!r} needs a simulator with a graphics stack: unavailable on this box")
    return make


ENV_ADAPTERS: Dict[str, Callable] = {"reach": ReachEnv, **{n: _unavailable(n) for n in
                                                            ("libero", "calvin", "simpler_env", "robotwin", "maniskill")}}


@dataclasses.dataclass
class EvalConfig:
    env: str = "reach"
    env_kwargs: dict = dataclasses.field(default_factory=dict)
    episodes: int = 5                 # per task and seed
    replan_every: int = 4             # execute this many actions of a chunk before asking the policy again
    host: str = "127.0.0.1"
    port: int = 0
    output_dir: Optional[str] = None
    suite: str = "default"
    tasks: List[dict] = dataclasses.field(default_factory=list)   # [{"name": ..., "env_kwargs": {...}}]; empty: one task
    seeds: List[int] = dataclasses.field(default_factory=lambda: [0])
    resume: bool = True               # skip the episodes already in output_dir/results.jsonl
    min_episodes: int = 1             # floor checked in the report
    name: str = "run"


class ResourceMonitor:
    def __init__(self):
        import psutil

        self.proc = psutil.Process()
        self.samples: List[dict] = []

    def sample(self):
        self.samples.append({"rss_mb": self.proc.memory_info().rss / 2 ** 20, "cpu_percent": self.proc.cpu_percent(None)})

    def summary(self) -> dict:
        if not self.samples:
            return {}
        return {"rss_mb_max": max(s["rss_mb"] for s in self.samples),
                "cpu_percent_mean": float(np.mean([s["cpu_percent"] for s in self.samples]))}


def run_evaluation(cfg: EvalConfig, action_adapter: Optional[Callable[[np.ndarray, Observation], np.ndarray]] = None) -> dict:
    """Rolls out ``cfg.episodes`` episodes of every task and seed against the policy server at (host, port). Every finished
    episode is appended to ``output_dir/results.jsonl``; with ``resume`` the episodes found there are not run again. The
    report (``report.json`` / ``report.md`` / CSV summaries) covers old and new episodes. `action_adapter` maps a policy
    action and the current observation to the environment's command (identity by default)."""
    from . import metrics as M

    client = RPCClient(cfg.host, cfg.port)
    info = client.call("info")
    results = os.path.join(cfg.output_dir, "results.jsonl") if cfg.output_dir else None
    records = M.load_jsonl(results) if (results and cfg.resume) else []
    if results and not cfg.resume and os.path.isfile(results):
        os.remove(results)
    done = M.completed_keys(records)
    tasks = cfg.tasks or [{"name": cfg.env, "env_kwargs": cfg.env_kwargs}]
    mon = ResourceMonitor()
    for task_id, task in enumerate(tasks):
        for seed in cfg.seeds:
            kw = {**cfg.env_kwargs, **task.get("env_kwargs", {})}
            if "seed" not in kw:
                kw["seed"] = seed
            env = None
            for ep in range(cfg.episodes):
                key = (cfg.suite, task["name"], ep, seed)
                if env is None:
                    env = ENV_ADAPTERS[task.get("env", cfg.env)](**kw)
                obs = env.reset()              # also for finished episodes: the environment's random stream stays aligned
                if key in done:
                    continue
                finished, success, steps, rt, sv = False, False, 0, [], []
                while not finished:
                    t0 = time.perf_counter()
                    chunk = ActionChunk.from_wire(client.call("predict_action", observation=obs.to_wire()))
                    rt.append((time.perf_counter() - t0) * 1e3)
                    sv.append(client.last_server_ms)
                    for a in chunk.actions[:cfg.replan_every]:
                        cmd = action_adapter(a, obs) if action_adapter is not None else a
                        obs, finished, success = env.step(cmd)
                        steps += 1
                        if finished:
                            break
                    mon.sample()
                rec = {"suite": cfg.suite, "task": task["name"], "task_id": task_id, "episode": ep, "seed": seed,
                       "success": bool(success), "steps": steps, "failure_reason": None if success else "timeout",
                       "round_trip_ms": rt, "server_ms": sv}
                records.append(rec)
                if results:
                    M.append_jsonl(results, rec)
    client.close()
    cfg_dict = {k: v for k, v in dataclasses.asdict(cfg).items()}
    if cfg.output_dir:
        report = M.write_report(cfg.output_dir, records, name=cfg.name, policy=info, config=cfg_dict,
                                min_episodes=cfg.min_episodes, resources=mon.summary())
    else:
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            report = M.write_report(tmp, records, name=cfg.name, policy=info, config=cfg_dict, min_episodes=cfg.min_episodes,
                                    resources=mon.summary())
    report["env"] = cfg.env
    return report


def compare_reports(a: dict, b: dict) -> dict:
    """Differences between two reports (b - a) on the headline metrics."""
    return {"success_rate": b["success_rate"] - a["success_rate"], "mean_steps": b["mean_steps"] - a["mean_steps"],
            "latency_ms_mean": b["latency_ms"]["mean"] - a["latency_ms"]["mean"]}
