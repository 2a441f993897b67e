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
    episodes: int = 5
    replan_every: int = 4  # execute this many actions of a chunk before asking the policy again
    host: str = "127.0.0.1"
    port: int = 0
    output_dir: Optional[str] = None


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
    """Rolls out `cfg.episodes` episodes against the policy server at (host, port). `action_adapter` maps a policy
    action and the current observation to the environment's command (identity by default)."""
    client = RPCClient(cfg.host, cfg.port)
    info = client.call("info")
    env = ENV_ADAPTERS[cfg.env](**cfg.env_kwargs)
    mon = ResourceMonitor()
    episodes, lat = [], []
    for _ in range(cfg.episodes):
        obs, done, success, steps = env.reset(), False, False, 0
        while not done:
            t0 = time.perf_counter()
            chunk = ActionChunk.from_wire(client.call("predict_action", observation=obs.to_wire()))
            lat.append({"round_trip_ms": (time.perf_counter() - t0) * 1e3, "server_ms": client.last_server_ms})
            for a in chunk.actions[:cfg.replan_every]:
                cmd = action_adapter(a, obs) if action_adapter is not None else a
                obs, done, success = env.step(cmd)
                steps += 1
                if done:
                    break
            mon.sample()
        episodes.append({"success": success, "steps": steps})
    client.close()
    rt = np.array([x["round_trip_ms"] for x in lat])
    report = {"policy": info, "env": cfg.env, "episodes": episodes,
              "success_rate": float(np.mean([e["success"] for e in episodes])),
              "mean_steps": float(np.mean([e["steps"] for e in episodes])),
              "latency_ms": {"mean": float(rt.mean()), "p50": float(np.percentile(rt, 50)),
                             "p95": float(np.percentile(rt, 95)),
                             "server_mean": float(np.mean([x["server_ms"] for x in lat]))},
              "resources": mon.summary()}
    if cfg.output_dir:
        os.makedirs(cfg.output_dir, exist_ok=True)
        with open(os.path.join(cfg.output_dir, "report.json"), "w") as f:
            json.dump(report, f, indent=1)
    return report


def compare_reports(a: dict, b: dict) -> dict:
    """Differences between two reports (b - a) on the headline metrics."""
    return {"success_rate": b["success_rate"] - a["success_rate"], "mean_steps": b["mean_steps"] - a["mean_steps"],
            "latency_ms_mean": b["latency_ms"]["mean"] - a["latency_ms"]["mean"]}
