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


def transformed_payload(obs: Observation, transform, args, device="cpu", dtype=torch.float32):
    """The observation through the policy's TRAINING pipeline in inference mode (same resize mode, state normalisation,
    Pi0.5 prompt with the discretised state, embodiment / domain ids); returns the batch and the raw state (needed to turn
    relative actions back into absolute targets)."""
    cams = [obs.images[n].transpose(2, 0, 1).astype(np.float32) / 255.0 for n in sorted(obs.images)[:args.num_cameras]]
    while len(cams) < args.num_cameras:
        cams.append(np.zeros_like(cams[0]))
    hw = cams[0].shape[1:]
    cams = [c if c.shape[1:] == hw else np.zeros_like(cams[0]) for c in cams]
    raw_state = np.zeros(args.state_dim, np.float32)
    raw_state[:min(args.state_dim, obs.state.shape[0])] = obs.state[:args.state_dim]
    sample = {"images": np.stack(cams), "state": raw_state.copy(), "task": obs.instruction,
              "actions": np.zeros((args.action_horizon, args.action_dim), np.float32),
              "action_mask": np.ones(args.action_horizon, np.float32)}
    if getattr(obs, "embodiment_tag", None):
        sample["embodiment_tag"] = sample["domain"] = obs.embodiment_tag
    out = transform(sample)
    if "text" not in out:
        out["text"] = hash_tokenize(obs.instruction, args.max_text_len)
    batch = {}
    for k, v in out.items():
        if k in ("actions", "action_mask"):
            continue
        t = torch.from_numpy(np.asarray(v))[None]
        batch[k] = t.to(device, dtype) if t.is_floating_point() else t.to(device)
    return batch, raw_state


class PolicyService:
    """``predict_action(observation) -> action chunk`` around a policy. With ``transform`` (the training pipeline built by
    ``embodied.transforms.build_transforms(args, stats, training=False)``) observations are prepared exactly as in training
    and predictions are returned in robot units."""

    def __init__(self, policy, args, action_space: str = "joint", denoise_steps: int = 10, transform=None):
        self.policy, self.args, self.space, self.steps = policy.eval(), args, action_space, denoise_steps
        self.device = next(policy.parameters()).device
        self.dtype = next(policy.parameters()).dtype
        self.calls = 0
        self.transform = transform

    @classmethod
    def from_output_dir(cls, policy, args, **kw):
        """Picks up ``stats.json`` written next to the checkpoints when the run used transforms."""
        import os
        transform = None
        path = os.path.join(args.output_dir, "stats.json")
        if getattr(args, "use_transforms", False) and os.path.isfile(path):
            from .. import transforms as T
            st = T.load_stats(path)
            st = {"state": st.get("state"), "actions": st.get("actions")}
            transform = T.build_transforms(args, {k: v for k, v in st.items() if v}, training=False)
        return cls(policy, args, transform=transform, **kw)

    def predict_action(self, observation: dict) -> dict:
        t0 = time.perf_counter()
        obs = Observation.from_wire(observation)
        a = self.args
        raw_state = None
        if self.transform is not None:
            batch, raw_state = transformed_payload(obs, self.transform, a, self.device, self.dtype)
        else:
            batch = PAYLOAD_BUILDERS.get(a.model_name, build_payload)(
                obs, image_size=a.image_size, num_cameras=a.num_cameras, max_text_len=a.max_text_len,
                state_dim=a.state_dim, device=self.device, dtype=self.dtype)
        actions = self.policy.predict_action(batch, steps=self.steps)[0].float().cpu().numpy()
        if self.transform is not None:
            from ..transforms import NormalizeStateAction
            nsa = self.transform.find(NormalizeStateAction)
            if nsa is not None:
                actions = nsa.unnormalize_actions(actions[:, :a.action_dim], raw_state)
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
