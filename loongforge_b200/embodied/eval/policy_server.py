"""Policy server: wraps a trained policy behind the RPC transport with a ``predict_action`` method; payload builders
turn protocol observations into model batches; a mock policy serves tests and dry runs (reference:
loongforge/embodied/eval/servers/loongforge_server.py, predict_action_interface.py, payload_builders/*, mock server)."""
from __future__ import annotations

import time
from typing import Callable, Dict, Optional

import numpy as np
import torch

from ..data import hash_tokenize
from .protocol import ActionChunk, Observation
from .transport import RPCServer


def build_payload(obs: Observation, *, image_size: int, num_cameras: int, max_text_len: int, state_dim: int,
                  device="cpu", dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Protocol observation -> model batch of size 1: images resized (nearest) to the training size, scaled to [0, 1],
    CHW; state padded / cut to `state_dim`; instruction tokenised."""
    cams = []
    for name in sorted(obs.images)[:num_cameras]:
        img = obs.images[name]
        ys = (np.arange(image_size) * img.shape[0] / image_size).astype(int)
        xs = (np.arange(image_size) * img.shape[1] / image_size).astype(int)
        cams.append(img[ys][:, xs].transpose(2, 0, 1).astype(np.float32) / 255.0)
    while len(cams) < num_cameras:
        cams.append(np.zeros_like(cams[0]))
    state = np.zeros(state_dim, np.float32)
    state[:min(state_dim, obs.state.shape[0])] = obs.state[:state_dim]
    return {"images": torch.from_numpy(np.stack(cams))[None].to(device, dtype),
            "state": torch.from_numpy(state)[None].to(device, dtype),
            "text": torch.from_numpy(hash_tokenize(obs.instruction, max_text_len))[None].to(device)}


PAYLOAD_BUILDERS: Dict[str, Callable] = {n: build_payload for n in
                                         ("pi05", "groot_n1_6", "groot_n1_7", "xvla", "lingbot_va", "fastwam",
                                          "dreamzero", "cosmos3")}


class PolicyService:
    """``predict_action(observation) -> action chunk`` around a FlowMatchingPolicy."""

    def __init__(self, policy, args, action_space: str = "joint", denoise_steps: int = 10):
        self.policy, self.args, self.space, self.steps = policy.eval(), args, action_space, denoise_steps
        self.device = next(policy.parameters()).device
        self.dtype = next(policy.parameters()).dtype
        self.calls = 0

    def predict_action(self, observation: dict) -> dict:
        t0 = time.perf_counter()
        obs = Observation.from_wire(observation)
        a = self.args
        batch = PAYLOAD_BUILDERS.get(a.model_name, build_payload)(
            obs, image_size=a.image_size, num_cameras=a.num_cameras, max_text_len=a.max_text_len,
            state_dim=a.state_dim, device=self.device, dtype=self.dtype)
        actions = self.policy.predict_action(batch, steps=self.steps)[0].float().cpu().numpy()
        self.calls += 1
        return ActionChunk(actions, self.space, (time.perf_counter() - t0) * 1e3).to_wire()

    def info(self) -> dict:
        return {"model": self.args.model_name, "action_space": self.space, "horizon": self.args.action_horizon,
                "action_dim": self.args.action_dim, "calls": self.calls}


class MockPolicyService:
    """Deterministic stand-in: action t of the chunk is ``state[:action_dim] * 0 + (step + t) * 0.01``."""

    def __init__(self, horizon: int = 8, action_dim: int = 7, action_space: str = "joint"):
        self.h, self.d, self.space, self.calls = horizon, action_dim, action_space, 0

    def predict_action(self, observation: dict) -> dict:
        obs = Observation.from_wire(observation)
        self.calls += 1
        base = (obs.step + np.arange(self.h, dtype=np.float32))[:, None] * 0.01
        return ActionChunk(np.repeat(base, self.d, 1), self.space, 0.0).to_wire()

    def info(self) -> dict:
        return {"model": "mock", "action_space": self.space, "horizon": self.h, "action_dim": self.d, "calls": self.calls}


def serve(service, host: str = "127.0.0.1", port: int = 0) -> RPCServer:
    srv = RPCServer(host, port)
    srv.register("predict_action", service.predict_action)
    srv.register("info", service.info)
    return srv.start()
