"""Per-sample transforms of the embodied data sets (numpy, so they run inside data-loader workers) and the per-policy
pipelines built from them.

* ``Normalizer``           — state / action normalisation with data-set statistics: ``mean_std``, ``min_max`` and ``q99``
  (1st / 99th percentile) to [-1, 1] with clipping, ``scale`` (by the largest magnitude), ``binary``; constant channels pass
  through (or map to 0); an optional channel mask leaves channels such as a gripper command untouched; ``inverse`` takes
  predictions back to robot units. ``compute_stats`` gathers the statistics in one pass, ``save_stats`` / ``load_stats`` use
  the ``stats.json`` layout of LeRobot data sets (``{key: {mean, std, min, max, q01, q99}}``).
* images                   — ``resize_with_pad`` (aspect kept, black borders), ``center_crop_resize``, ``ImageAugment`` (random
  crop + resize back, small rotation, brightness / contrast / saturation jitter; the same geometric draw for all cameras
  of a sample when ``shared`` is set).
* action representation    — ``to_relative`` / ``to_absolute`` (actions as offsets from the current state for the masked
  channels), ``RotationTransform`` between euler / quaternion / rotation matrix / 6-D.
* policy pipelines (``build_transforms``): Pi0.5 writes the normalised state, discretised into 256 bins, into the prompt
  (``Task: ..., State: 12 200 ...;\\nAction: ``) and pads actions to the model width; GR00T maps an embodiment tag to its
  id and concatenates per-part state / action vectors in a fixed order; DreamZero clips min-max normalised values to
  [-1, 1] and marks samples without real actions; Cosmos3 adds the domain id, the number of real action channels and
  appends the robot description to the caption.

(reference: loongforge/embodied/data/datasets/transforms/utils/image_transform.py:27-285, pi05/transforms/pi05_transform.py:27-293,
dreamzero/transforms/state_action.py:22-566, groot_n1_6/transforms/groot_transform.py, cosmos3/transforms/cosmos3_action_transform.py:162-408)
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

import numpy as np

from .eval import action_decoders as AD

Sample = Dict[str, Any]


# ------------------------------------------------------------------------------------------------ statistics
class Normalizer:
    MODES = ("mean_std", "min_max", "q99", "scale", "binary", "identity")

    def __init__(self, mode: str, stats: Dict[str, Sequence[float]], mask: Optional[Sequence[bool]] = None):
        if mode not in self.MODES:
            raise ValueError(f"unknown normalisation mode {mode!r}; known: {self.MODES}")
        self.mode = mode
        self.s = {k: np.asarray(v, dtype=np.float32) for k, v in stats.items()}
        self.mask = None if mask is None else np.asarray(mask, dtype=bool)
        need = {"mean_std": ("mean", "std"), "min_max": ("min", "max"), "q99": ("q01", "q99"), "scale": ("min", "max")}.get(mode, ())
        missing = [k for k in need if k not in self.s]
        if missing:
            raise KeyError(f"normalisation mode {mode!r} needs the statistics {missing}")

    def _range(self):
        return (self.s["q01"], self.s["q99"]) if self.mode == "q99" else (self.s["min"], self.s["max"])

    def forward(self, x: np.ndarray) -> np.ndarray:
        x = np.asarray(x, dtype=np.float32)
        if self.mode == "identity":
            return x
        if self.mode == "binary":
            y = (x > 0.5).astype(np.float32)
        elif self.mode == "mean_std":
            std = self.s["std"]
            y = np.where(std != 0, (x - self.s["mean"]) / np.where(std != 0, std, 1), x)
        elif self.mode == "scale":
            m = np.maximum(np.abs(self.s["min"]), np.abs(self.s["max"]))
            y = np.where(m != 0, x / np.where(m != 0, m, 1), 0.0)
        else:
            lo, hi = self._range()
            live = lo != hi
            y = np.where(live, 2 * (x - lo) / np.where(live, hi - lo, 1) - 1, x if self.mode == "q99" else 0.0)
            y = np.clip(y, -1.0, 1.0) if self.mode == "min_max" else np.where(live, np.clip(y, -1.0, 1.0), y)
        return (np.where(self.mask, y, x) if self.mask is not None else y).astype(np.float32)

    def inverse(self, y: np.ndarray) -> np.ndarray:
        y = np.asarray(y, dtype=np.float32)
        if self.mode == "identity":
            return y
        if self.mode == "binary":
            x = (y > 0.5).astype(np.float32)
        elif self.mode == "mean_std":
            x = np.where(self.s["std"] != 0, y * self.s["std"] + self.s["mean"], y)
        elif self.mode == "scale":
            x = y * np.maximum(np.abs(self.s["min"]), np.abs(self.s["max"]))
        else:
            lo, hi = self._range()
            x = np.where(lo != hi, (y + 1) / 2 * (hi - lo) + lo, y if self.mode == "q99" else lo)
        return (np.where(self.mask, x, y) if self.mask is not None else x).astype(np.float32)


def compute_stats(rows: Iterable[np.ndarray]) -> Dict[str, List[float]]:
    """mean / std / min / max / q01 / q99 per channel over all rows (each ``[..., D]``)."""
    data = np.concatenate([np.asarray(r, dtype=np.float64).reshape(-1, np.asarray(r).shape[-1]) for r in rows], axis=0)
    return {"mean": data.mean(0).tolist(), "std": data.std(0).tolist(), "min": data.min(0).tolist(), "max": data.max(0).tolist(),
            "q01": np.quantile(data, 0.01, axis=0).tolist(), "q99": np.quantile(data, 0.99, axis=0).tolist(), "count": [int(data.shape[0])]}


def dataset_stats(dataset, keys=("state", "actions"), limit: Optional[int] = None, relative_mask=None) -> Dict[str, Dict[str, List[float]]]:
    """Statistics of the first ``limit`` samples; with ``relative_mask`` the actions are taken relative to the state first
    (the statistics must describe what is normalised)."""
    n = len(dataset) if limit is None else min(limit, len(dataset))
    rows: Dict[str, List[np.ndarray]] = {k: [] for k in keys}
    for i in range(n):
        s = dataset[i]
        if relative_mask:
            s = dict(s, actions=to_relative(s["actions"], s["state"], relative_mask))
        for k in keys:
            rows[k].append(np.asarray(s[k]))
    return {k: compute_stats(v) for k, v in rows.items()}


def save_stats(stats: dict, path: str) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        json.dump(stats, f)


def merge_stats(parts: Sequence[dict]) -> dict:
    """Statistics of the union from statistics of the parts (per episode, per data set): for every feature the pooled mean
    and standard deviation (weighted by ``count``; the variance of a union is the weighted mean of the parts' variances
    plus the spread of their means), the overall min / max, and for the quantiles the outermost of the parts' values (an
    upper bound of the spread: exact quantiles cannot be merged). (reference: loongforge/embodied/data/datasets/
    compute_stats.py:32-92)"""
    out = {}
    for key in sorted({k for p in parts for k in p}):
        have = [p[key] for p in parts if key in p]
        n = np.array([float(np.asarray(h.get("count", [1])).reshape(-1)[0]) for h in have])
        mean = np.stack([np.asarray(h["mean"], dtype=np.float64) for h in have])
        var = np.stack([np.asarray(h["std"], dtype=np.float64) ** 2 for h in have])
        w = n.reshape(-1, *([1] * (mean.ndim - 1))) / n.sum()
        pooled = (mean * w).sum(0)
        merged = {"mean": pooled.tolist(), "std": np.sqrt(((var + (mean - pooled) ** 2) * w).sum(0)).tolist(),
                  "min": np.min(np.stack([np.asarray(h["min"], dtype=np.float64) for h in have]), 0).tolist(),
                  "max": np.max(np.stack([np.asarray(h["max"], dtype=np.float64) for h in have]), 0).tolist(),
                  "count": [int(n.sum())]}
        if all("q01" in h and "q99" in h for h in have):
            merged["q01"] = np.min(np.stack([np.asarray(h["q01"], dtype=np.float64) for h in have]), 0).tolist()
            merged["q99"] = np.max(np.stack([np.asarray(h["q99"], dtype=np.float64) for h in have]), 0).tolist()
        out[key] = merged
    return out


def load_stats(path: str) -> dict:
    """``stats.json`` of a data set, or the directory holding ``meta/stats.json``; a LeRobot v2.1 directory that only has
    per-episode statistics (``meta/episodes_stats.jsonl``, one ``{"episode_index", "stats"}`` record per line) is merged."""
    if os.path.isdir(path):
        whole, per_episode = os.path.join(path, "meta", "stats.json"), os.path.join(path, "meta", "episodes_stats.jsonl")
        if not os.path.isfile(whole) and os.path.isfile(per_episode):
            with open(per_episode) as f:
                return merge_stats([json.loads(line)["stats"] for line in f if line.strip()])
        path = whole
    with open(path) as f:
        return json.load(f)


# ------------------------------------------------------------------------------------------------ images
def _resize(img: np.ndarray, h: int, w: int) -> np.ndarray:
    """Bilinear resize of ``[C, H, W]`` (float) with half-pixel centres."""
    C, H, W = img.shape
    if (H, W) == (h, w):
        return img
    ys = np.clip((np.arange(h) + 0.5) * H / h - 0.5, 0, H - 1)
    xs = np.clip((np.arange(w) + 0.5) * W / w - 0.5, 0, W - 1)
    y0, x0 = np.floor(ys).astype(int), np.floor(xs).astype(int)
    y1, x1 = np.minimum(y0 + 1, H - 1), np.minimum(x0 + 1, W - 1)
    wy, wx = (ys - y0)[None, :, None], (xs - x0)[None, None, :]
    top = img[:, y0][:, :, x0] * (1 - wx) + img[:, y0][:, :, x1] * wx
    bot = img[:, y1][:, :, x0] * (1 - wx) + img[:, y1][:, :, x1] * wx
    return (top * (1 - wy) + bot * wy).astype(img.dtype)


def resize_with_pad(img: np.ndarray, h: int, w: int, fill: float = 0.0) -> np.ndarray:
    """Aspect-preserving resize into an ``h x w`` canvas, centred, borders filled."""
    C, H, W = img.shape
    r = min(h / H, w / W)
    nh, nw = max(1, round(H * r)), max(1, round(W * r))
    out = np.full((C, h, w), fill, dtype=img.dtype)
    top, left = (h - nh) // 2, (w - nw) // 2
    out[:, top:top + nh, left:left + nw] = _resize(img, nh, nw)
    return out


def center_crop_resize(img: np.ndarray, h: int, w: int, crop_fraction: float = 1.0) -> np.ndarray:
    """Largest centred window with the target aspect (shrunk by ``crop_fraction``), resized to ``h x w``."""
    C, H, W = img.shape
    r = min(H / h, W / w) * crop_fraction
    ch, cw = max(1, int(h * r)), max(1, int(w * r))
    top, left = (H - ch) // 2, (W - cw) // 2
    return _resize(img[:, top:top + ch, left:left + cw], h, w)


class ImageAugment:
    """Training-time augmentation of ``images [cams, C, H, W]`` in [0, 1]."""

    def __init__(self, crop_scale: float = 0.95, rotate_deg: float = 5.0, brightness: float = 0.3, contrast: float = 0.4,
                 saturation: float = 0.5, shared: bool = True, seed: Optional[int] = None):
        self.crop_scale, self.rotate_deg = crop_scale, rotate_deg
        self.brightness, self.contrast, self.saturation, self.shared = brightness, contrast, saturation, shared
        self.rng = np.random.default_rng(seed)

    def _draw(self):
        r = self.rng
        return dict(scale=self.crop_scale, off=r.random(2), angle=np.deg2rad(r.uniform(-self.rotate_deg, self.rotate_deg)),
                    b=1 + r.uniform(-self.brightness, self.brightness), c=1 + r.uniform(-self.contrast, self.contrast),
                    s=1 + r.uniform(-self.saturation, self.saturation))

    @staticmethod
    def _rotate(img, angle):
        if abs(angle) < 1e-6:
            return img
        C, H, W = img.shape
        yy, xx = np.meshgrid(np.arange(H) - (H - 1) / 2, np.arange(W) - (W - 1) / 2, indexing="ij")
        sy = np.cos(angle) * yy + np.sin(angle) * xx + (H - 1) / 2
        sx = -np.sin(angle) * yy + np.cos(angle) * xx + (W - 1) / 2
        inside = (sy >= 0) & (sy <= H - 1) & (sx >= 0) & (sx <= W - 1)
        y0, x0 = np.clip(np.round(sy).astype(int), 0, H - 1), np.clip(np.round(sx).astype(int), 0, W - 1)
        return img[:, y0, x0] * inside[None]

    def _one(self, img, d):
        C, H, W = img.shape
        ch, cw = max(1, int(H * d["scale"])), max(1, int(W * d["scale"]))
        top, left = int(d["off"][0] * (H - ch + 1)), int(d["off"][1] * (W - cw + 1))
        img = _resize(img[:, top:top + ch, left:left + cw], H, W)
        img = self._rotate(img, d["angle"])
        img = img * d["b"]
        mean = img.mean()
        img = (img - mean) * d["c"] + mean
        if C == 3:
            gray = img.mean(0, keepdims=True)
            img = (img - gray) * d["s"] + gray
        return np.clip(img, 0.0, 1.0).astype(np.float32)

    def __call__(self, sample: Sample) -> Sample:
        imgs = np.asarray(sample["images"], dtype=np.float32)
        d = self._draw()
        out = []
        for cam in imgs:
            out.append(self._one(cam, d))
            if not self.shared:
                d = self._draw()
        sample["images"] = np.stack(out)
        return sample


class ResizeImages:
    def __init__(self, size: int, mode: str = "pad"):
        assert mode in ("pad", "crop", "stretch")
        self.size, self.mode = size, mode

    def __call__(self, sample: Sample) -> Sample:
        f = {"pad": resize_with_pad, "crop": center_crop_resize, "stretch": _resize}[self.mode]
        for key in ("images", "video"):
            if key in sample:
                arr = np.asarray(sample[key], dtype=np.float32)
                sample[key] = np.stack([f(a, self.size, self.size) for a in arr])
        return sample


# ------------------------------------------------------------------------------------------------ actions
def to_relative(actions: np.ndarray, state: np.ndarray, mask: Sequence[bool]) -> np.ndarray:
    """Masked action channels become offsets from the current state (same channel order as the state's first dims)."""
    m = np.asarray(mask, dtype=bool)
    out = np.array(actions, dtype=np.float32)
    out[..., m] -= np.asarray(state, dtype=np.float32)[..., :out.shape[-1]][..., m]
    return out


def to_absolute(actions: np.ndarray, state: np.ndarray, mask: Sequence[bool]) -> np.ndarray:
    m = np.asarray(mask, dtype=bool)
    out = np.array(actions, dtype=np.float32)
    out[..., m] += np.asarray(state, dtype=np.float32)[..., :out.shape[-1]][..., m]
    return out


class RotationTransform:
    """Between ``euler`` (xyz, 3), ``quat`` (wxyz, 4), ``matrix`` (9, row-major) and ``rot6d`` (6) through rotation matrices."""

    DIMS = {"euler": 3, "quat": 4, "matrix": 9, "rot6d": 6}

    def __init__(self, src: str, dst: str):
        assert src in self.DIMS and dst in self.DIMS
        self.src, self.dst = src, dst

    @staticmethod
    def _to_matrix(x, rep):
        if rep == "euler":
            return np.stack([AD.euler_to_matrix(v) for v in x.reshape(-1, 3)]).reshape(*x.shape[:-1], 3, 3)
        if rep == "quat":
            return AD.quat_to_matrix(x)
        if rep == "rot6d":
            return AD.rot6d_to_matrix(x)
        return x.reshape(*x.shape[:-1], 3, 3)

    @staticmethod
    def _from_matrix(R, rep):
        if rep == "euler":
            sy = np.clip(-R[..., 2, 0], -1, 1)
            return np.stack([np.arctan2(R[..., 2, 1], R[..., 2, 2]), np.arcsin(sy), np.arctan2(R[..., 1, 0], R[..., 0, 0])], -1)
        if rep == "quat":
            return AD.matrix_to_quat(R)
        if rep == "rot6d":
            return AD.matrix_to_rot6d(R)
        return R.reshape(*R.shape[:-2], 9)

    def forward(self, x: np.ndarray) -> np.ndarray:
        return self._from_matrix(self._to_matrix(np.asarray(x, dtype=np.float64), self.src), self.dst).astype(np.float32)

    def inverse(self, x: np.ndarray) -> np.ndarray:
        return self._from_matrix(self._to_matrix(np.asarray(x, dtype=np.float64), self.dst), self.src).astype(np.float32)


class NormalizeStateAction:
    def __init__(self, stats: dict, mode: str = "q99", action_mask: Optional[Sequence[bool]] = None, relative_mask=None):
        self.state = Normalizer(mode, stats["state"]) if "state" in stats else None
        self.action = Normalizer(mode, stats["actions"], action_mask) if "actions" in stats else None
        self.relative_mask = relative_mask

    def __call__(self, sample: Sample) -> Sample:
        if self.relative_mask is not None:
            sample["actions"] = to_relative(sample["actions"], sample["state"], self.relative_mask)
        if self.state is not None:
            sample["state"] = self.state.forward(sample["state"])
        if self.action is not None:
            sample["actions"] = self.action.forward(sample["actions"])
        return sample

    def unnormalize_actions(self, actions: np.ndarray, raw_state: Optional[np.ndarray] = None) -> np.ndarray:
        """Model output -> robot units (and back to absolute targets when the data were relative)."""
        a = self.action.inverse(actions) if self.action is not None else np.asarray(actions, dtype=np.float32)
        if self.relative_mask is not None and raw_state is not None:
            a = to_absolute(a, raw_state, self.relative_mask)
        return a


class Pad:
    """Pads ``state`` / ``actions`` channels with zeros up to the model's widths (``action_dim_mask`` marks the real ones)."""

    def __init__(self, state_dim: Optional[int] = None, action_dim: Optional[int] = None):
        self.sd, self.ad = state_dim, action_dim

    def __call__(self, sample: Sample) -> Sample:
        if self.sd and sample["state"].shape[-1] < self.sd:
            sample["state"] = np.pad(sample["state"], [(0, 0)] * (sample["state"].ndim - 1) + [(0, self.sd - sample["state"].shape[-1])])
        if self.ad:
            A = sample["actions"].shape[-1]
            sample["action_dim_mask"] = (np.arange(self.ad) < A).astype(np.float32)
            if A < self.ad:
                sample["actions"] = np.pad(sample["actions"], [(0, 0), (0, self.ad - A)])
        return sample


# ------------------------------------------------------------------------------------------------ policies
class Pi05Prompt:
    """Normalised state -> ``num_bins`` bins on [-1, 1] -> ``Task: <task>, State: <bins>;\\nAction: `` tokenised into ``text``."""

    def __init__(self, tokenize: Callable[[str, int], np.ndarray], max_len: int, num_bins: int = 256, max_state_dim: Optional[int] = None,
                 template: str = "Task: {task}, State: {state};\nAction: "):
        self.tokenize, self.max_len, self.bins, self.max_state_dim, self.template = tokenize, max_len, num_bins, max_state_dim, template

    def prompt(self, task: str, state: Optional[np.ndarray]) -> str:
        task = task.strip().replace("_", " ").replace("\n", " ")
        if state is None:
            return f"Task: {task};\nAction: "
        s = np.asarray(state, dtype=np.float32).reshape(-1)
        d = self.max_state_dim or s.shape[0]
        s = np.pad(s, (0, max(d - s.shape[0], 0)))[:d]
        edges = np.linspace(-1, 1, self.bins + 1)[:-1]
        return self.template.format(task=task, state=" ".join(map(str, np.digitize(s, edges) - 1)))

    def __call__(self, sample: Sample) -> Sample:
        sample["prompt"] = self.prompt(sample.get("task", "perform the task"), sample.get("state"))
        sample["text"] = self.tokenize(sample["prompt"], self.max_len)
        return sample


class GrootEmbodiment:
    """Embodiment tag -> id; per-part state / action dictionaries concatenated in the order of ``state_keys`` / ``action_keys``."""

    def __init__(self, tags: Dict[str, int], default_tag: str = "new_embodiment", state_keys: Sequence[str] = (), action_keys: Sequence[str] = ()):
        self.tags, self.default = dict(tags), default_tag
        self.state_keys, self.action_keys = list(state_keys), list(action_keys)
        if default_tag not in self.tags:
            self.tags[default_tag] = max(self.tags.values(), default=-1) + 1

    def __call__(self, sample: Sample) -> Sample:
        sample["embodiment_id"] = np.int64(self.tags.get(sample.get("embodiment_tag", self.default), self.tags[self.default]))
        if self.state_keys and isinstance(sample.get("state"), dict):
            sample["state"] = np.concatenate([np.asarray(sample["state"][k], np.float32).reshape(-1) for k in self.state_keys])
        if self.action_keys and isinstance(sample.get("actions"), dict):
            sample["actions"] = np.concatenate([np.asarray(sample["actions"][k], np.float32) for k in self.action_keys], axis=-1)
        return sample


class DreamZeroFlags:
    """Values already min-max normalised are clipped to [-1, 1]; samples whose action mask is empty are marked
    ``has_real_action = 0`` (video-only supervision)."""

    def __call__(self, sample: Sample) -> Sample:
        sample["actions"] = np.clip(sample["actions"], -1.0, 1.0).astype(np.float32)
        sample["state"] = np.clip(sample["state"], -1.0, 1.0).astype(np.float32)
        m = sample.get("action_mask")
        sample["has_real_action"] = np.float32(1.0 if m is None or float(np.sum(m)) > 0 else 0.0)
        return sample


class Cosmos3Meta:
    """Domain id, number of real action channels, and the robot description appended to the caption."""

    def __init__(self, domains: Dict[str, int], default_domain: str = "default", description: Optional[str] = None,
                 tokenize: Optional[Callable[[str, int], np.ndarray]] = None, max_len: int = 64):
        self.domains, self.default, self.description = dict(domains), default_domain, description
        self.domains.setdefault(default_domain, max(self.domains.values(), default=-1) + 1)
        self.tokenize, self.max_len = tokenize, max_len

    @staticmethod
    def append_sentence(caption: str, addition: str) -> str:
        caption = caption.strip()
        if not addition:
            return caption
        if caption and caption[-1] not in ".!?":
            caption += "."
        return (caption + " " + addition.strip()).strip()

    def __call__(self, sample: Sample) -> Sample:
        sample["domain_id"] = np.int64(self.domains.get(sample.get("domain", self.default), self.domains[self.default]))
        sample["raw_action_dim"] = np.int64(sample["actions"].shape[-1])
        if self.description and self.tokenize is not None and "task" in sample:
            sample["caption"] = self.append_sentence(sample["task"], self.description)
            sample["text"] = self.tokenize(sample["caption"], self.max_len)
        return sample


class Compose:
    def __init__(self, steps: Sequence[Callable[[Sample], Sample]]):
        self.steps = list(steps)

    def __call__(self, sample: Sample) -> Sample:
        for s in self.steps:
            sample = s(sample)
        # strings and nested values do not collate: the tensors of the batch are what remains
        return {k: v for k, v in sample.items() if isinstance(v, (np.ndarray, np.generic, int, float))}

    def find(self, cls):
        return next((s for s in self.steps if isinstance(s, cls)), None)


def build_transforms(args, stats: Optional[dict] = None, training: bool = True, tokenize=None) -> Compose:
    """The pipeline of ``args.model_name``: resize, (training) augmentation, normalisation, then the policy's own step."""
    from .data import hash_tokenize
    tokenize = tokenize or (lambda text, n: hash_tokenize(text, n))
    name = args.model_name
    steps: List[Callable] = [ResizeImages(args.image_size, getattr(args, "image_resize_mode", "pad"))]
    if training and getattr(args, "image_augmentation", False):
        steps.append(ImageAugment(seed=getattr(args, "seed", None)))
    if stats:
        mode = getattr(args, "normalization_mode", None) or ("min_max" if name == "dreamzero" else "q99" if name in ("pi05", "xvla") else "mean_std")
        steps.append(NormalizeStateAction(stats, mode, relative_mask=getattr(args, "relative_action_mask", None) or None))
    if name == "pi05":
        steps.append(Pi05Prompt(tokenize, args.max_text_len, max_state_dim=args.state_dim))
    elif name.startswith("groot"):
        steps.append(GrootEmbodiment(getattr(args, "embodiment_tags", None) or {"new_embodiment": 0}))
    elif name == "dreamzero":
        steps += [GrootEmbodiment(getattr(args, "embodiment_tags", None) or {"new_embodiment": 0}), DreamZeroFlags()]
    elif name == "cosmos3":
        steps.append(Cosmos3Meta(getattr(args, "embodiment_tags", None) or {"default": 0}, description=getattr(args, "robot_description", None),
                                 tokenize=tokenize, max_len=args.max_text_len))
    return Compose(steps)
