"""Wire schema between environment adapters and policy servers (reference: loongforge/embodied/eval/protocol/schema.py)."""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional

import numpy as np

PROTOCOL_VERSION = 1


@dataclasses.dataclass
class Observation:
    images: Dict[str, np.ndarray]  # camera name -> uint8 [H, W, 3]
    state: np.ndarray  # float32 [state_dim]
    instruction: str
    episode_id: int = 0
    step: int = 0

    def to_wire(self) -> dict:
        return {"v": PROTOCOL_VERSION, "images": self.images, "state": self.state.astype(np.float32),
                "instruction": self.instruction, "episode_id": int(self.episode_id), "step": int(self.step)}

    @staticmethod
    def from_wire(d: dict) -> "Observation":
        validate_observation(d)
        return Observation(d["images"], np.asarray(d["state"], np.float32), d["instruction"], d.get("episode_id", 0),
                           d.get("step", 0))


@dataclasses.dataclass
class ActionChunk:
    actions: np.ndarray  # float32 [horizon, action_dim]
    action_space: str = "joint"  # joint | ee_delta_quat | ee_delta_6d | ee_delta_euler
    latency_ms: Optional[float] = None

    def to_wire(self) -> dict:
        return {"v": PROTOCOL_VERSION, "actions": self.actions.astype(np.float32), "action_space": self.action_space,
                "latency_ms": self.latency_ms}

    @staticmethod
    def from_wire(d: dict) -> "ActionChunk":
        if d.get("v") != PROTOCOL_VERSION:
            raise ValueError(f"protocol version {d.get('v')} != {PROTOCOL_VERSION}")
        a = np.asarray(d["actions"], np.float32)
        if a.ndim != 2:
            raise ValueError("actions must be [horizon, action_dim]")
        return ActionChunk(a, d.get("action_space", "joint"), d.get("latency_ms"))


def validate_observation(d: dict) -> None:
    if d.get("v") != PROTOCOL_VERSION:
        raise ValueError(f"protocol version {d.get('v')} != {PROTOCOL_VERSION}")
    if not isinstance(d.get("images"), dict) or not d["images"]:
        raise ValueError("observation needs at least one camera image")
    for name, img in d["images"].items():
        if not (isinstance(img, np.ndarray) and img.ndim == 3 and img.shape[2] == 3 and img.dtype == np.uint8):
            raise ValueError(f"image {name!r} must be uint8 [H, W, 3]")
    if np.asarray(d.get("state")).ndim != 1:
        raise ValueError("state must be a vector")
    if not isinstance(d.get("instruction"), str):
        raise ValueError("instruction must be a string")
