"""Datasets and collators of the embodied stack.

Every sample is one time step of an episode: camera images, a proprioceptive state, a language instruction and the
chunk of the next ``action_horizon`` actions (padded at episode end, with a mask); with ``video_frames > 0`` also the
camera-0 frames of the coming steps (``video [T, 3, H, W]``), which the world-model policies encode into latents. Sources:

* ``SyntheticEpisodes``  — deterministic random episodes (benchmarks, tests);
* ``NpzEpisodes``        — a directory of ``episode_*.npz`` files (arrays ``images [T, cams, C, H, W]``, ``state``,
  ``actions``, optional ``task``);
* ``hdf5_data.HDF5Episodes`` — bimanual end-effector episodes in HDF5 files, re-sampled into two-second action windows
  (reference: hdf5_dataset.py);
* ``LeRobotParquet``     — LeRobot-style ``data/chunk-*/episode_*.parquet`` tables with ``observation.state``,
  ``action``, ``episode_index``, ``task_index`` columns plus ``meta/tasks.jsonl`` (reference: lerobot_dataset.py).

(reference: loongforge/embodied/data/dataloader.py, data/datasets/lerobot_dataset.py, hdf5_dataset.py)
"""
from __future__ import annotations

import glob
import json
import os
import zlib
from typing import Dict, List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, DistributedSampler


def _chunk(actions: np.ndarray, t: int, horizon: int):
    seg = actions[t:t + horizon]
    n = seg.shape[0]
    mask = np.zeros(horizon, dtype=np.float32)
    mask[:n] = 1.0
    if n < horizon:
        seg = np.concatenate([seg, np.repeat(seg[-1:], horizon - n, 0)], 0)
    return seg.astype(np.float32), mask


def _future_frames(frames_at, t: int, length: int, n: int, stride: int) -> np.ndarray:
    """``[n, 3, H, W]``: camera-0 frames at steps t, t + stride, ... (the last frame repeats past the episode's end)."""
    return np.stack([frames_at(min(t + i * stride, length - 1)) for i in range(n)]).astype(np.float32)


def hash_tokenize(text: str, max_len: int, vocab: int = 32000) -> np.ndarray:
    """Whitespace tokens hashed into a fixed vocabulary (stand-in for the model tokenizer in tests / synthetic runs)."""
    ids = [(zlib.crc32(w.encode()) % (vocab - 2)) + 2 for w in text.lower().split()][:max_len]
    return np.array(ids + [0] * (max_len - len(ids)), dtype=np.int64)


class SyntheticEpisodes(Dataset):
    raw = False  # True: samples also carry the task string (and other non-tensor fields) for the transforms

    def __init__(self, args, num_episodes: int = 8, episode_len: int = 32, seed: int = 0):
        self.a, self.n, self.L, self.seed = args, num_episodes, episode_len, seed

    def __len__(self):
        return self.n * self.L

    def __getitem__(self, i):
        a = self.a
        ep, t = divmod(i, self.L)
        rng = np.random.default_rng(self.seed * 100003 + ep)
        actions = rng.standard_normal((self.L, a.action_dim)).astype(np.float32).cumsum(0) * 0.1
        state = rng.standard_normal((self.L, a.state_dim)).astype(np.float32)
        img = np.random.default_rng(i).random((a.num_cameras, 3, a.image_size, a.image_size), dtype=np.float32)
        chunk, mask = _chunk(actions, t, a.action_horizon)
        task = f"task {ep % 3} move the object"
        out = {"images": img, "state": state[t], "actions": chunk, "action_mask": mask,
               "text": hash_tokenize(task, a.max_text_len)}
        if self.raw:
            out["task"] = task
        if getattr(a, "video_frames", 0):
            # a smooth drift of the current image: frame k is the image rolled by k pixels (something a world model can learn)
            out["video"] = _future_frames(lambda k: np.roll(img[0], k - t, axis=-1), t, self.L + a.video_frames * a.video_frame_stride,
                                          a.video_frames, a.video_frame_stride)
        return out


class NpzEpisodes(Dataset):
    raw = False

    def __init__(self, args, path: str):
        self.a = args
        self.files = sorted(glob.glob(os.path.join(path, "episode_*.npz")))
        if not self.files:
            raise FileNotFoundError(f"no episode_*.npz under {path}")
        self.index = []
        for fi, f in enumerate(self.files):
            with np.load(f, allow_pickle=False) as z:
                self.index += [(fi, t) for t in range(z["actions"].shape[0])]
        self._cache = (None, None)

    def __len__(self):
        return len(self.index)

    def _episode(self, fi):
        if self._cache[0] != fi:
            with np.load(self.files[fi], allow_pickle=False) as z:
                self._cache = (fi, {k: z[k] for k in z.files})
        return self._cache[1]

    def __getitem__(self, i):
        fi, t = self.index[i]
        ep = self._episode(fi)
        chunk, mask = _chunk(ep["actions"], t, self.a.action_horizon)
        task = str(ep["task"]) if "task" in ep else "do the task"
        out = {"images": ep["images"][t].astype(np.float32), "state": ep["state"][t].astype(np.float32),
               "actions": chunk, "action_mask": mask, "text": hash_tokenize(task, self.a.max_text_len)}
        if self.raw:
            out["task"] = task
            if "embodiment_tag" in ep:
                out["embodiment_tag"] = out["domain"] = str(ep["embodiment_tag"])
        if getattr(self.a, "video_frames", 0):
            out["video"] = _future_frames(lambda k: ep["images"][k][0], t, ep["images"].shape[0], self.a.video_frames,
                                          self.a.video_frame_stride)
        return out


class LeRobotParquet(Dataset):
    """LeRobot v2 layout:

    * ``meta/info.json``      fps, robot type, ``data_path`` / ``video_path`` templates, ``features`` (which keys are videos);
    * ``meta/tasks.jsonl``    task index -> instruction; ``meta/episodes.jsonl`` episode lengths; ``meta/stats.json`` statistics;
    * ``data/chunk-XXX/episode_XXXXXX.parquet``  one row per step: ``observation.state``, ``action``, ``task_index``, ...
      (image columns holding encoded bytes are decoded when present);
    * ``videos/chunk-XXX/<camera key>/episode_XXXXXX.mp4``  one video per camera and episode, decoded by frame index with
      OpenCV (a few captures stay open per worker).

    ``cameras`` picks / orders the camera keys (default: the first ``num_cameras`` video features); ``episodes`` restricts
    the episode indices; without videos and image columns the images are zeros (state-only data sets)."""

    raw = False

    def __init__(self, args, path: str, cameras: Optional[List[str]] = None, episodes: Optional[List[int]] = None):
        import pyarrow.parquet as pq

        self.a, self.root = args, path
        info_p = os.path.join(path, "meta", "info.json")
        self.info = json.load(open(info_p)) if os.path.isfile(info_p) else {}
        files = sorted(glob.glob(os.path.join(path, "data", "chunk-*", "episode_*.parquet")))
        if not files:
            raise FileNotFoundError(f"no LeRobot parquet episodes under {path}")
        self.tasks: Dict[int, str] = {}
        tp = os.path.join(path, "meta", "tasks.jsonl")
        if os.path.isfile(tp):
            with open(tp) as f:
                for line in f:
                    if line.strip():
                        r = json.loads(line)
                        self.tasks[int(r["task_index"])] = r["task"]
        feats = self.info.get("features", {})
        video_keys = [k for k, v in feats.items() if v.get("dtype") == "video"]
        image_keys = [k for k, v in feats.items() if v.get("dtype") == "image"]
        self.cameras = list(cameras or (video_keys + image_keys))[:args.num_cameras]
        self.video_keys = set(video_keys)
        self.robot = self.info.get("robot_type")
        self.episodes, self.index = [], []
        for f in files:
            ep_idx = int(os.path.basename(f).split("_")[1].split(".")[0])
            if episodes is not None and ep_idx not in episodes:
                continue
            t = pq.read_table(f).to_pydict()
            ep = {"index": ep_idx, "chunk": os.path.basename(os.path.dirname(f)),
                  "state": np.asarray(t["observation.state"], dtype=np.float32),
                  "actions": np.asarray(t["action"], dtype=np.float32),
                  "task": self.tasks.get(int(t["task_index"][0]), "") if "task_index" in t else "",
                  "frames": {k: t[k] for k in self.cameras if k in t and k not in self.video_keys}}
            self.index += [(len(self.episodes), i) for i in range(ep["actions"].shape[0])]
            self.episodes.append(ep)
        self._caps: Dict[str, object] = {}

    def __len__(self):
        return len(self.index)

    def stats(self) -> Optional[dict]:
        p = os.path.join(self.root, "meta", "stats.json")
        return json.load(open(p)) if os.path.isfile(p) else None

    def _video_file(self, ep: dict, key: str) -> str:
        tpl = self.info.get("video_path", "videos/{episode_chunk_dir}/{video_key}/episode_{episode_index:06d}.mp4")
        rel = tpl.format(episode_chunk=int(ep["chunk"].split("-")[1]), episode_chunk_dir=ep["chunk"], video_key=key,
                         episode_index=ep["index"])
        return os.path.join(self.root, rel)

    def _frame(self, ep: dict, key: str, t: int) -> np.ndarray:
        """``[3, H, W]`` in [0, 1] at the model's image size (nearest resize; the transforms resize properly when used)."""
        S = self.a.image_size
        img = None
        if key in ep["frames"]:
            cell = ep["frames"][key][t]
            data = cell.get("bytes") if isinstance(cell, dict) else cell
            import cv2
            img = cv2.imdecode(np.frombuffer(data, np.uint8), cv2.IMREAD_COLOR)[:, :, ::-1]
        elif key in self.video_keys and getattr(self.a, "video_backend", "opencv") != "opencv":
            from .video_backends import decode_frames
            f = self._video_file(ep, key)
            img = decode_frames(f, indices=[t], backend=self.a.video_backend)[0] if os.path.isfile(f) else None
        elif key in self.video_keys:
            import cv2
            f = self._video_file(ep, key)
            cap = self._caps.get(f)
            if cap is None and os.path.isfile(f):
                if len(self._caps) >= 8:
                    self._caps.pop(next(iter(self._caps))).release()
                cap = self._caps[f] = cv2.VideoCapture(f)
            if cap is not None:
                cap.set(cv2.CAP_PROP_POS_FRAMES, t)
                ok, fr = cap.read()
                img = fr[:, :, ::-1] if ok else None
        if img is None:
            return np.zeros((3, S, S), dtype=np.float32)
        ys = (np.arange(S) * img.shape[0] / S).astype(int)
        xs = (np.arange(S) * img.shape[1] / S).astype(int)
        return np.ascontiguousarray(img[ys][:, xs].transpose(2, 0, 1)).astype(np.float32) / 255.0

    def __getitem__(self, i):
        e, t = self.index[i]
        ep, a = self.episodes[e], self.a
        chunk, mask = _chunk(ep["actions"], t, a.action_horizon)
        cams = [self._frame(ep, k, t) for k in self.cameras]
        while len(cams) < a.num_cameras:
            cams.append(np.zeros((3, a.image_size, a.image_size), dtype=np.float32))
        out = {"images": np.stack(cams), "state": ep["state"][t], "actions": chunk, "action_mask": mask,
               "text": hash_tokenize(ep["task"], a.max_text_len)}
        if getattr(a, "video_frames", 0) and self.cameras:
            out["video"] = _future_frames(lambda k: self._frame(ep, self.cameras[0], k), t, ep["actions"].shape[0], a.video_frames,
                                          a.video_frame_stride)
        if self.raw:
            out["task"] = ep["task"]
            if self.robot:
                out["embodiment_tag"] = out["domain"] = str(self.robot)
        return out


LeRobotDataset = LeRobotParquet


def collate(samples: List[dict]) -> Dict[str, torch.Tensor]:
    return {k: torch.from_numpy(np.stack([s[k] for s in samples])) for k in samples[0]}


class TransformedDataset(Dataset):
    """A data set whose samples go through a ``transforms.Compose`` pipeline (in the worker that loads them)."""

    def __init__(self, base: Dataset, transform):
        base.raw = True
        self.base, self.transform = base, transform

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        return self.transform(self.base[i])


class PrecomputedFeatures(Dataset):
    """A data set whose samples take ``latents`` / ``text_emb`` / ``text_emb_mask`` / ``image_tokens`` from a cache written by
    ``tools/data_preprocess/embodied_precompute.py`` (same sample order) instead of carrying the raw video; the policies use
    these arrays in place of their codec, text encoder and image tower."""

    def __init__(self, base: Dataset, cache_dir: str):
        with open(os.path.join(cache_dir, "manifest.json")) as f:
            self.m = json.load(f)
        if not self.m.get("complete"):
            raise ValueError(f"{cache_dir}: the feature cache is not complete")
        if self.m["num_samples"] != len(base):
            raise ValueError(f"{cache_dir}: cache of {self.m['num_samples']} samples, data set of {len(base)}")
        self.base, self.dir = base, cache_dir
        self.firsts = np.array([s["first"] for s in self.m["shards"]])
        self._open = (None, None)

    @property
    def raw(self):
        return getattr(self.base, "raw", False)

    @raw.setter
    def raw(self, v):
        self.base.raw = v

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        s = int(np.searchsorted(self.firsts, i, side="right") - 1)
        if self._open[0] != s:
            with np.load(os.path.join(self.dir, self.m["shards"][s]["file"])) as z:
                self._open = (s, {k: z[k] for k in z.files})
        out = dict(self.base[i])
        out.pop("video", None)
        j = i - int(self.firsts[s])
        for k, arr in self._open[1].items():
            out[k] = arr[j].astype(np.float32) if arr.dtype.kind == "f" else arr[j]
        return out


class MixtureDataset(Dataset):
    """Several data sets (other robots, other tasks) sampled in fixed proportions: an epoch has ``length`` samples, sample
    i comes from data set ``schedule[i]`` (drawn once from the weights with the seed), walking each data set in its own order
    and wrapping around the small ones. Every sample carries ``dataset_id``."""

    def __init__(self, datasets: List[Dataset], weights: Optional[List[float]] = None, seed: int = 0, length: Optional[int] = None):
        assert datasets
        self.sets = datasets
        w = np.asarray(weights or [len(d) for d in datasets], dtype=np.float64)
        self.weights = w / w.sum()
        self.n = int(length or sum(len(d) for d in datasets))
        rng = np.random.default_rng(seed)
        self.schedule = rng.choice(len(datasets), size=self.n, p=self.weights)
        self.local = np.zeros(self.n, dtype=np.int64)
        for k in range(len(datasets)):
            pos = np.nonzero(self.schedule == k)[0]
            self.local[pos] = np.arange(len(pos)) % max(len(datasets[k]), 1)

    @property
    def raw(self):
        return all(getattr(d, "raw", False) for d in self.sets)

    @raw.setter
    def raw(self, v):
        for d in self.sets:
            d.raw = v

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        k = int(self.schedule[i])
        out = dict(self.sets[k][int(self.local[i])])
        out["dataset_id"] = np.int64(k)
        return out


def _base_dataset(args) -> Dataset:
    mix = getattr(args, "dataset_mixture", None)
    if mix:
        import copy
        sets, weights = [], []
        for entry in mix:
            sub = copy.copy(args)
            sub.dataset_mixture = None
            sub.dataset_type, sub.dataset_path = entry.get("type", args.dataset_type), entry.get("path")
            sets.append(_base_dataset(sub))
            weights.append(float(entry.get("weight", len(sets[-1]))))
        return MixtureDataset(sets, weights, seed=args.seed, length=getattr(args, "mixture_epoch_length", None))
    if args.dataset_type == "synthetic":
        return SyntheticEpisodes(args)
    if args.dataset_type == "npz_episodes":
        return NpzEpisodes(args, args.dataset_path)
    if args.dataset_type == "hdf5":
        from .hdf5_data import HDF5Episodes
        return HDF5Episodes(args, args.dataset_path)
    if args.dataset_type == "lerobot":
        return LeRobotParquet(args, args.dataset_path)
    raise ValueError(args.dataset_type)


def build_dataset(args, training: bool = True) -> Dataset:
    """The data set of ``args.dataset_type``; with ``use_transforms`` wrapped in the policy's pipeline, with statistics from
    ``stats_path`` or, failing that, computed over the first ``stats_samples`` samples and kept as ``output_dir/stats.json``
    (the file an evaluation server reads to turn predictions back into robot units)."""
    ds = _base_dataset(args)
    if getattr(args, "precomputed_cache", None):
        ds = PrecomputedFeatures(ds, args.precomputed_cache)
    if not getattr(args, "use_transforms", False):
        return ds
    from . import transforms as T
    own = os.path.join(args.output_dir, "stats.json")
    if args.stats_path:
        stats = T.load_stats(args.stats_path)
    elif os.path.isfile(own):
        stats = T.load_stats(own)
    else:
        stats = T.dataset_stats(ds, limit=args.stats_samples, relative_mask=list(args.relative_action_mask) or None)
        if int(os.environ.get("RANK", "0")) == 0:
            T.save_stats(stats, own)
    stats = {"state": stats.get("state", stats.get("observation.state")), "actions": stats.get("actions", stats.get("action"))}
    return TransformedDataset(ds, T.build_transforms(args, {k: v for k, v in stats.items() if v}, training))


class BlockShardSampler(torch.utils.data.Sampler):
    """The epoch's (shuffled) order is cut into batches first and whole batches go to the ranks in turn: the ranks' k-th
    batches together are ``world`` consecutive batches of the one-process order, so a run on N ranks with batch B sees the
    batches a one-process run with batch B sees, N at a time (``DistributedSampler`` deals single samples instead).
    (reference: loongforge/embodied/data/datasets/sampler_builder.py:47-112)"""

    def __init__(self, dataset, batch_size: int, num_replicas: int, rank: int, shuffle: bool = True, seed: int = 0):
        self.n, self.b, self.world, self.rank, self.shuffle, self.seed, self.epoch = len(dataset), batch_size, num_replicas, rank, shuffle, seed, 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __len__(self) -> int:                                 # only rounds in which every rank gets a whole batch
        return self.n // (self.b * self.world) * self.b

    def __iter__(self):
        order = (torch.randperm(self.n, generator=torch.Generator().manual_seed(self.seed + self.epoch)).tolist()
                 if self.shuffle else list(range(self.n)))
        for r in range(self.n // (self.b * self.world)):
            at = (r * self.world + self.rank) * self.b
            yield from order[at:at + self.b]


class ResumableLoader:
    """DataLoader + sampler whose position (epoch, batches consumed) can be saved and restored. ``sampler``:
    ``distributed`` (samples dealt to ranks one by one) or ``block_shard`` (whole batches dealt to ranks)."""

    def __init__(self, dataset: Dataset, batch_size: int, rank: int, world: int, seed: int, num_workers: int = 0,
                 sampler: str = "distributed"):
        if sampler == "block_shard":
            self.sampler = BlockShardSampler(dataset, batch_size, world, rank, shuffle=True, seed=seed)
        elif sampler == "distributed":
            self.sampler = DistributedSampler(dataset, num_replicas=world, rank=rank, shuffle=True, seed=seed, drop_last=True)
        else:
            raise ValueError(f"unknown sampler {sampler!r} (distributed | block_shard)")
        self.loader = DataLoader(dataset, batch_size=batch_size, sampler=self.sampler, collate_fn=collate,
                                 num_workers=num_workers, drop_last=True, pin_memory=torch.cuda.is_available())
        self.epoch, self.consumed = 0, 0

    def state_dict(self):
        return {"epoch": self.epoch, "consumed": self.consumed}

    def load_state_dict(self, sd):
        self.epoch, self.consumed = sd["epoch"], sd["consumed"]

    def __iter__(self):
        while True:
            self.sampler.set_epoch(self.epoch)
            skip = self.consumed
            for i, batch in enumerate(self.loader):
                if i < skip:
                    continue
                self.consumed = i + 1
                yield batch
            self.epoch, self.consumed = self.epoch + 1, 0
