"""Bimanual end-effector episodes stored as HDF5 files (the layout X-VLA is fine-tuned on).

Directory::

    metadata.json                    optional: dataset_name, datalist (episode files), observation_key (camera data sets),
                                     language_instruction_key
    episode_<n>.hdf5                 observations/eef_quaternion [T, 16] = per arm xyz (3), quaternion xyzw (4), gripper (1)
                                     observations/eef_left_time, observations/eef_right_time [T] seconds (optional: 30 Hz)
                                     observations/images/<camera> [T, H, W, 3] uint8 (or encoded image bytes per step)
                                     language_instruction

A sample starts at every second step that leaves 30 steps of trajectory; both arms are re-sampled on a common clock over the
next two seconds at ``action_horizon + 1`` points of (xyz, 6-D rotation, gripper closed) per arm: the first point is the
state, the rest are the actions (absolute end-effector targets, 20 numbers). Windows in which neither arm moves are
dropped. Images are read per sample, one frame per camera.

Files are opened through ``opener`` (default: ``h5py.File``); anything that maps data-set paths to arrays works, which is how
the trajectory logic is tested without the HDF5 library.

(reference: loongforge/embodied/data/datasets/hdf5_dataset.py:52-623)
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Callable, Dict, List, Optional

import numpy as np
from torch.utils.data import Dataset

from .data import _future_frames, hash_tokenize

RATE_HZ = 30.0          # when the file holds no time stamps
WINDOW_S = 2.0          # the action window
MARGIN, STRIDE = 30, 2  # steps kept free at the end of an episode; distance between sample starts
STATIC_EPS = 1e-5


def quat_xyzw_to_rot6d(q: np.ndarray) -> np.ndarray:
    """``[..., 4]`` -> ``[..., 6]``: the first two columns of the rotation matrix, row by row."""
    q = np.asarray(q, dtype=np.float64)
    q = q / np.maximum(np.linalg.norm(q, axis=-1, keepdims=True), 1e-12)
    x, y, z, w = q[..., 0], q[..., 1], q[..., 2], q[..., 3]
    c0 = np.stack([1 - 2 * (y * y + z * z), 2 * (x * y + z * w), 2 * (x * z - y * w)], axis=-1)   # first column
    c1 = np.stack([2 * (x * y - z * w), 1 - 2 * (x * x + z * z), 2 * (y * z + x * w)], axis=-1)   # second column
    return np.stack([c0, c1], axis=-1).reshape(*q.shape[:-1], 6)


def arm_trajectories(eef: np.ndarray):
    """``[T, 16]`` -> left, right ``[T, 10]``: xyz, 6-D rotation, gripper closed (opening x 50 below 1)."""
    eef = np.asarray(eef)
    arms = []
    for o in (0, 8):
        closed = (eef[:, o + 7:o + 8] * 50 < 1.0).astype(np.float32)
        arms.append(np.concatenate([eef[:, o:o + 3], quat_xyzw_to_rot6d(eef[:, o + 3:o + 7]), closed], axis=-1).astype(np.float32))
    return arms[0], arms[1]


def resample(times: np.ndarray, values: np.ndarray, query: np.ndarray) -> np.ndarray:
    """Linear interpolation of every channel at ``query`` (held at the ends)."""
    return np.stack([np.interp(query, times, values[:, c]) for c in range(values.shape[1])], axis=-1).astype(np.float32)


def _open_h5(path: str):
    try:
        import h5py
    except ImportError as e:  # pragma: no cover - depends on the installation
        raise ImportError("dataset_type=hdf5 needs the h5py package (or pass an opener that maps data-set paths to arrays)") from e
    return h5py.File(path, "r")


def _episode_number(path: str) -> int:
    m = re.search(r"(\d+)$", os.path.splitext(os.path.basename(path))[0])
    return int(m.group(1)) if m else 0


class HDF5Episodes(Dataset):
    raw = False

    def __init__(self, args, path: str, opener: Optional[Callable] = None, pattern: str = "episode_*.hdf5"):
        self.a, self.root, self.opener = args, path, opener or _open_h5
        self.meta = self._metadata(path)
        files = self.meta.get("datalist") or sorted(glob.glob(os.path.join(path, pattern)), key=_episode_number)
        self.files = [f if os.path.isabs(f) else os.path.join(path, f) for f in files]
        if not self.files:
            raise FileNotFoundError(f"no {pattern} under {path}")
        self.cameras = list(self.meta.get("observation_key") or ["observations/images/cam_high"])[:args.num_cameras]
        self.text_key = self.meta.get("language_instruction_key", "language_instruction")
        self.robot = self.meta.get("dataset_name")
        self._open: Dict[int, object] = {}
        self.episodes = [self._episode_tables(i) for i in range(len(self.files))]
        self.index = [(e, t) for e, ep in enumerate(self.episodes)
                      for t in range(0, max(0, ep["steps"] - MARGIN), STRIDE) if not self._static(ep, t)]

    @staticmethod
    def _metadata(root: str) -> dict:
        cands = [os.path.join(root, "metadata.json")] + sorted(glob.glob(os.path.join(root, "*.json")))
        for p in cands:
            if os.path.isfile(p):
                with open(p) as f:
                    meta = json.load(f)
                if p.endswith("metadata.json") or ("dataset_name" in meta and "datalist" in meta):
                    return meta
        return {}

    def _file(self, e: int):
        f = self._open.get(e)
        if f is None:
            if len(self._open) >= 8:                      # a few episodes stay open per worker
                old = self._open.pop(next(iter(self._open)))
                getattr(old, "close", lambda: None)()
            f = self._open[e] = self.opener(self.files[e])
        return f

    def _episode_tables(self, e: int) -> dict:
        f = self._file(e)
        left, right = arm_trajectories(f["observations/eef_quaternion"][()])
        clock = lambda key, n: (np.asarray(f[key][()], dtype=np.float64) if key in f else np.arange(n) / RATE_HZ)
        lt, rt = clock("observations/eef_left_time", len(left)), clock("observations/eef_right_time", len(right))
        text = f[self.text_key] if self.text_key in f else "do the task"
        text = text[()] if hasattr(text, "shape") else text        # a scalar data set, or the string itself
        text = text.decode() if isinstance(text, bytes) else str(text)
        ref = (lt + rt) / 2
        return {"left": left, "right": right, "lt": lt, "rt": rt, "ref": ref, "end": float(ref.max()), "steps": len(left),
                "task": text, "cameras": [k for k in self.cameras if k in f]}

    def _window(self, ep: dict, t: int) -> np.ndarray:
        """``[horizon + 1, 20]``: both arms on the common clock from step ``t`` over the next two seconds."""
        now = ep["ref"][t]
        q = np.linspace(now, min(now + WINDOW_S, ep["end"]), self.a.action_horizon + 1)
        return np.concatenate([resample(ep["lt"], ep["left"], q), resample(ep["rt"], ep["right"], q)], axis=-1)

    def _static(self, ep: dict, t: int) -> bool:
        w = self._window(ep, t)
        return bool(np.abs(w[1] - w[0]).max() < STATIC_EPS)

    def _frame(self, e: int, key: str, t: int) -> np.ndarray:
        """``[3, S, S]`` in [0, 1] (nearest resize; the transforms resize properly when used)."""
        S = self.a.image_size
        raw = np.asarray(self._file(e)[key][t])
        if raw.ndim == 1 or raw.dtype.kind in "SOV":       # an encoded image
            import cv2
            raw = cv2.imdecode(np.frombuffer(raw.tobytes() if raw.ndim else bytes(raw[()]), np.uint8), cv2.IMREAD_COLOR)[:, :, ::-1]
        if raw.shape[0] in (1, 3) and raw.shape[-1] not in (1, 3):
            raw = raw.transpose(1, 2, 0)
        img = raw.astype(np.float32) / (255.0 if raw.dtype == np.uint8 or raw.max() > 1.5 else 1.0)
        ys = (np.arange(S) * img.shape[0] / S).astype(int)
        xs = (np.arange(S) * img.shape[1] / S).astype(int)
        return np.ascontiguousarray(img[ys][:, xs].transpose(2, 0, 1))

    def __len__(self):
        return len(self.index)

    def __getitem__(self, i):
        e, t = self.index[i]
        ep, a = self.episodes[e], self.a
        traj = self._window(ep, t)
        cams = [self._frame(e, k, t) for k in ep["cameras"]]
        while len(cams) < a.num_cameras:
            cams.append(np.zeros((3, a.image_size, a.image_size), dtype=np.float32))
        out = {"images": np.stack(cams), "state": traj[0], "actions": traj[1:],
               "action_mask": np.ones(a.action_horizon, dtype=np.float32), "text": hash_tokenize(ep["task"], a.max_text_len)}
        if getattr(a, "video_frames", 0) and ep["cameras"]:
            out["video"] = _future_frames(lambda k: self._frame(e, ep["cameras"][0], k), t, ep["steps"], a.video_frames,
                                          a.video_frame_stride)
        if self.raw:
            out["task"] = ep["task"]
            if self.robot:
                out["embodiment_tag"] = out["domain"] = str(self.robot)
        return out

    def __getstate__(self):
        state = dict(self.__dict__)
        state["_open"] = {}                                # file handles do not travel to loader workers
        return state
