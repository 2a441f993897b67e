"""Multimodal sample encoding, online packing and sequence padding for VLM training.

A raw sample is ``{"images": [uint8 HWC arrays], "conversation": [{"role", "content"}]}`` where the user content
carries ``<image>`` markers. Task encoders turn it into model inputs: pixel patches (flattened
``C x t x p x p``), ``grid_thw``, token ids with every marker expanded to ``n_patches / merge^2`` image tokens,
labels masked outside assistant turns. The online packer fills fixed-length buffers greedily (first-fit-decreasing)
and emits ``cu_seqlens``; sequences are padded to the multiple that TP / CP / FP8 need (reference:
loongforge/data/multimodal/** task encoders, online packer, dataloader_provider.py:36-185)."""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

IGNORE = -100


@dataclasses.dataclass
class VisionPreprocess:
    patch_size: int = 14
    temporal_patch_size: int = 2
    merge_size: int = 2
    min_pixels: int = 56 * 56
    max_pixels: int = 14 * 14 * 4 * 1280
    mean: Sequence[float] = (0.48145466, 0.4578275, 0.40821073)
    std: Sequence[float] = (0.26862954, 0.26130258, 0.27577711)

    def smart_resize(self, h: int, w: int):
        """Round both sides to a multiple of patch * merge, keeping the area within [min_pixels, max_pixels]."""
        f = self.patch_size * self.merge_size
        hb, wb = max(f, round(h / f) * f), max(f, round(w / f) * f)
        if hb * wb > self.max_pixels:
            beta = math.sqrt(h * w / self.max_pixels)
            hb, wb = max(f, math.floor(h / beta / f) * f), max(f, math.floor(w / beta / f) * f)
        elif hb * wb < self.min_pixels:
            beta = math.sqrt(self.min_pixels / (h * w))
            hb, wb = math.ceil(h * beta / f) * f, math.ceil(w * beta / f) * f
        return hb, wb

    def __call__(self, image: np.ndarray):
        """uint8 [H, W, 3] -> (patches [n, C*t*p*p] fp32, grid (t, h, w)). A still image is repeated over the
        temporal patch."""
        H, W = image.shape[:2]
        hb, wb = self.smart_resize(H, W)
        ys = (np.arange(hb) * H / hb).astype(int)
        xs = (np.arange(wb) * W / wb).astype(int)
        img = image[ys][:, xs].astype(np.float32) / 255.0
        img = (img - np.asarray(self.mean, np.float32)) / np.asarray(self.std, np.float32)
        chw = np.repeat(img.transpose(2, 0, 1)[None], self.temporal_patch_size, 0)  # [t, C, H, W]
        p, m = self.patch_size, self.merge_size
        gh, gw = hb // p, wb // p
        x = chw.reshape(1, self.temporal_patch_size, 3, gh // m, m, p, gw // m, m, p)
        # patches ordered in merge units: (grid_t, gh/m, gw/m, m, m) x (C, t, p, p)
        x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gh * gw, 3 * self.temporal_patch_size * p * p)
        return x, (1, gh, gw)


class VLMTaskEncoder:
    """Conversation + images -> tokens / labels / pixels. ``tokenize(text) -> List[int]``."""

    def __init__(self, tokenize, image_token_id: int, vision: Optional[VisionPreprocess] = None,
                 image_marker: str = "<image>", roles=("user", "assistant"), eos_id: Optional[int] = None):
        self.tok, self.img_id, self.vision = tokenize, image_token_id, vision or VisionPreprocess()
        self.marker, self.roles, self.eos = image_marker, roles, eos_id

    def encode(self, sample: Dict) -> Dict[str, torch.Tensor]:
        images = list(sample.get("images", []))
        pix, grids, ids, labels = [], [], [], []
        k = 0
        for turn in sample["conversation"]:
            parts = turn["content"].split(self.marker)
            t_ids: List[int] = []
            for j, part in enumerate(parts):
                if part:
                    t_ids += self.tok(part)
                if j < len(parts) - 1:
                    p, g = self.vision(images[k])
                    k += 1
                    pix.append(p)
                    grids.append(g)
                    t_ids += [self.img_id] * (p.shape[0] // self.vision.merge_size ** 2)
            if turn["role"] == self.roles[1]:
                if self.eos is not None:
                    t_ids.append(self.eos)
                labels += t_ids
            else:
                labels += [IGNORE] * len(t_ids)
            ids += t_ids
        if k != len(images):
            raise ValueError(f"{len(images)} images but {k} markers")
        tokens = torch.tensor(ids, dtype=torch.long)
        lab = torch.tensor(labels[1:] + [IGNORE], dtype=torch.long)  # next-token targets
        return {"tokens": tokens, "labels": lab.clamp(min=0), "loss_mask": (lab != IGNORE).float(),
                "pixels": torch.from_numpy(np.concatenate(pix)) if pix else torch.zeros(0, 0),
                "grid_thw": torch.tensor(grids, dtype=torch.long).view(-1, 3)}


def pad_to_multiple(n: int, tp: int = 1, cp: int = 1, sequence_parallel: bool = False, fp8: bool = False) -> int:
    """Sequence lengths must divide by 2*cp (load-balanced CP chunks), by tp under sequence parallelism and by 16 for
    FP8 GEMM rows."""
    m = 1
    if cp > 1:
        m = math.lcm(m, 2 * cp)
    if sequence_parallel and tp > 1:
        m = math.lcm(m, tp * (2 * cp if cp > 1 else 1))
    if fp8:
        m = math.lcm(m, 16)
    return (n + m - 1) // m * m


class OnlinePacker:
    """Buffers encoded samples and emits packs of at most `seq_len` tokens (first-fit decreasing over the buffer)."""

    def __init__(self, seq_len: int, buffer_size: int = 64, pad_id: int = 0, pad_to_seq_len: bool = False, **pad_kw):
        """``pad_to_seq_len``: every pack is padded to exactly `seq_len` tokens (fixed shapes for pipeline stages)."""
        self.L, self.buf_size, self.pad_id, self.pad_kw = seq_len, buffer_size, pad_id, pad_kw
        self.pad_full = pad_to_seq_len
        self.buf: List[Dict[str, torch.Tensor]] = []

    def add(self, sample: Dict[str, torch.Tensor]) -> List[Dict[str, torch.Tensor]]:
        if sample["tokens"].numel() > self.L:
            return []  # over-long samples are dropped, as the reference's packer does
        self.buf.append(sample)
        return self._emit() if len(self.buf) >= self.buf_size else []

    def flush(self) -> List[Dict[str, torch.Tensor]]:
        out = []
        while self.buf:
            out += self._emit(force=True)
        return out

    def _emit(self, force: bool = False) -> List[Dict[str, torch.Tensor]]:
        self.buf.sort(key=lambda s: -s["tokens"].numel())
        bins: List[List[Dict]] = []
        room: List[int] = []
        for s in self.buf:
            n = s["tokens"].numel()
            for i, r in enumerate(room):
                if n <= r:
                    bins[i].append(s)
                    room[i] -= n
                    break
            else:
                bins.append([s])
                room.append(self.L - n)
        # keep the emptiest bin in the buffer (it may still fill up) unless flushing
        keep = [] if force or len(bins) == 1 else [max(range(len(bins)), key=lambda i: room[i])]
        self.buf = [s for i in keep for s in bins[i]]
        return [self._pack(b) for i, b in enumerate(bins) if i not in keep]

    def _pack(self, samples: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        lens = [s["tokens"].numel() for s in samples]
        total = self.L if self.pad_full else pad_to_multiple(sum(lens), **self.pad_kw)
        pad = total - sum(lens)
        cat = lambda k, fill, dt: torch.cat([s[k] for s in samples] + [torch.full((pad,), fill, dtype=dt)])  # noqa: E731
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        if pad:
            cu.append(total)  # padding forms its own (masked) sequence so attention never crosses into it
        pix = [s["pixels"] for s in samples if s["pixels"].numel()]
        return {"tokens": cat("tokens", self.pad_id, torch.long), "labels": cat("labels", 0, torch.long),
                "loss_mask": cat("loss_mask", 0.0, torch.float32),
                # per-sequence text positions, or the samples' own 3-row (t, h, w) multimodal positions
                "position_ids": (torch.cat([s["mrope"] for s in samples] + [torch.arange(pad).expand(3, -1)], dim=1)
                                 if all("mrope" in s for s in samples)
                                 else torch.cat([torch.arange(n) for n in lens] + [torch.arange(pad)])),
                "cu_seqlens": torch.tensor(cu, dtype=torch.int32),
                "pixels": torch.cat(pix) if pix else torch.zeros(0, 0),
                "grid_thw": torch.cat([s["grid_thw"] for s in samples]) if pix else torch.zeros(0, 3, dtype=torch.long)}


# ----------------------------------------------------------------------------- reading shards, building micro-batches
def decode_image(data: bytes, ext: str) -> np.ndarray:
    """Image file bytes -> uint8 HWC array (``.npy`` arrays pass through)."""
    import io

    if ext.endswith("npy"):
        return np.load(io.BytesIO(data))
    from PIL import Image
    return np.asarray(Image.open(io.BytesIO(data)).convert("RGB"))


def is_packed_dataset(root: str) -> bool:
    """True for shards written by tools/data_preprocess/vlm_offline_packing.py (packs decided offline)."""
    import json
    import os
    with open(os.path.join(root, "index.json")) as f:
        return bool(json.load(f).get("packed"))


VIDEO_EXTENSIONS = ("mp4", "avi", "mov", "mkv", "webm")


def decode_video(data: bytes, ext: str = "mp4", frame_num: Optional[int] = None, fps: Optional[float] = None) -> List[np.ndarray]:
    """Frames ``[H, W, 3]`` uint8 of an encoded video: every frame, or frames sampled at ``fps`` (of the video's own clock),
    thinned evenly to at most ``frame_num`` (``--frame-num`` / ``--fps``). OpenCV reads files, so the bytes pass through
    a temporary file."""
    import os
    import tempfile

    import cv2
    fd, path = tempfile.mkstemp(suffix="." + ext.split(".")[-1])
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(data)
        cap = cv2.VideoCapture(path)
        total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        native = cap.get(cv2.CAP_PROP_FPS) or 0.0
        if total <= 0:
            raise ValueError("video has no frames")
        step = max(native / fps, 1.0) if (fps and native > 0) else 1.0
        want = [min(int(round(i * step)), total - 1) for i in range(int((total - 1) // step) + 1)]
        if frame_num and len(want) > frame_num:
            want = [want[int(round(i * (len(want) - 1) / max(frame_num - 1, 1)))] for i in range(frame_num)]
        frames, nxt = [], 0
        for idx in sorted(set(want)):
            if idx != nxt:
                cap.set(cv2.CAP_PROP_POS_FRAMES, idx)
            ok, fr = cap.read()
            nxt = idx + 1
            if ok:
                frames.append(np.ascontiguousarray(fr[:, :, ::-1]))
        cap.release()
        if not frames:
            raise ValueError("no frame could be decoded")
        return frames
    finally:
        os.remove(path)


def webdataset_samples(root: str, *, dp_rank: int = 0, dp_size: int = 1, seed: int = 0, start_sample: int = 0,
                       epochs: Optional[int] = None, frame_num: Optional[int] = None, fps: Optional[float] = None):
    """Raw samples (``{"images": [...], "conversation": [...]}``) from the tar shards under `root` (the layout written
    by tools/data_preprocess/vlm_to_webdataset.py: ``index.json`` + ``shard-*.tar`` with ``{key}.json`` and
    ``{key}[.n].{ext}`` members). Shards are visited in a per-epoch shuffled order that all ranks share; rank r keeps
    every dp_size-th sample (every dp_size-th PACK of shards packed offline, whose members stay together).
    ``start_sample`` skips what an earlier run of this rank consumed. Members with a video extension are decoded into
    frame lists (``videos``), sampled with ``frame_num`` / ``fps``."""
    import json
    import os
    import tarfile

    with open(os.path.join(root, "index.json")) as f:
        idx = json.load(f)
    shards = [os.path.join(root, sh["name"]) for sh in idx["shards"]]
    packed = bool(idx.get("packed"))  # packs decided offline: the unit handed to a rank is a whole pack
    n, epoch = 0, 0
    while epochs is None or epoch < epochs:
        order = np.random.RandomState(seed + epoch).permutation(len(shards))
        for si in order:
            cur, group, last_pack = None, {}, None

            def emit(group, meta):
                members = sorted((k for k in group if k != "json"), key=lambda k: (len(k), k))
                vids = [k for k in members if k.split(".")[-1].lower() in VIDEO_EXTENSIONS]
                imgs = [k for k in members if k not in vids]
                pack = {"pack_id": meta["pack_id"], "pack_size": meta["pack_size"]} if "pack_id" in meta else {}
                conv = meta.get("conversation") or [
                    {"role": "user" if c.get("from", c.get("role")) in ("human", "user") else "assistant",
                     "content": c.get("value", c.get("content", ""))} for c in meta.get("conversations", [])]
                out = {"images": [decode_image(group[k], k) for k in imgs], "conversation": conv, **pack}
                if vids:  # video members become frame lists for the <video> markers of the conversation
                    out["videos"] = [decode_video(group[k], k, frame_num, fps) for k in vids]
                return out

            def take(group):
                """Counts the sample (or, for packed shards, its pack) and says whether this rank keeps it."""
                nonlocal n, last_pack
                meta = json.loads(group["json"])
                if packed and meta.get("pack_id") == last_pack:
                    unit = n - 1  # another member of the pack counted last
                else:
                    unit, n = n, n + 1
                    last_pack = meta.get("pack_id") if packed else None
                keep = unit % dp_size == dp_rank and unit // dp_size >= start_sample
                return emit(group, meta) if keep else None

            with tarfile.open(shards[si]) as tar:
                for m in tar:
                    key, _, ext = m.name.partition(".")
                    if key != cur and cur is not None:
                        out = take(group)
                        if out is not None:
                            yield out
                        group = {}
                    cur = key
                    group[ext] = tar.extractfile(m).read()
                if cur is not None:
                    out = take(group)
                    if out is not None:
                        yield out
        epoch += 1


def merge_video_into_image_stream(enc: Dict, image_id: int, video_id: Optional[int]) -> Dict:
    """The model scatters vision-tower features into the image placeholders in order. A sample with videos therefore gets
    ONE patch stream and ONE grid list in the order the media appear in its tokens (``media_order``), and its video
    placeholders are renamed to the image placeholder — after the position ids were computed from the original ids."""
    if "video_pixels" not in enc:
        return enc
    pix, grids = enc["pixels"], enc["grid_thw"]
    vpix, vgrids = enc["video_pixels"], enc["video_grid_thw"]
    i_off = [0] + torch.cumsum(grids.prod(-1), 0).tolist() if len(grids) else [0]
    v_off = [0] + torch.cumsum(vgrids.prod(-1), 0).tolist()
    parts, out_grids, ki, kv = [], [], 0, 0
    for kind in enc["media_order"].tolist():
        if kind == 0:
            parts.append(pix[i_off[ki]:i_off[ki + 1]])
            out_grids.append(grids[ki])
            ki += 1
        else:
            parts.append(vpix[v_off[kv]:v_off[kv + 1]].to(pix.dtype if pix.numel() else vpix.dtype))
            out_grids.append(vgrids[kv])
            kv += 1
    enc = dict(enc)
    enc["pixels"], enc["grid_thw"] = torch.cat(parts), torch.stack(out_grids)
    if video_id is not None and video_id != image_id:
        enc["tokens"] = torch.where(enc["tokens"] == video_id, torch.full_like(enc["tokens"], image_id), enc["tokens"])
    for k in ("video_pixels", "video_grid_thw", "media_order"):
        enc.pop(k)
    return enc


def vlm_batch_iterator(samples, encoder: VLMTaskEncoder, seq_len: int, *, merge_size: int = 2, pad_id: int = 0,
                       packing: bool = True, buffer_size: int = 16, pin_memory: bool = False):
    """Raw samples -> micro-batches of the vision-language trainer: one packed row of exactly `seq_len` tokens with
    ``cu_seqlens``, 3-row multimodal position ids, the row's image patches and grids."""
    from .position_ids import mrope_ids

    packer = OnlinePacker(seq_len, buffer_size=buffer_size if packing else 1, pad_id=pad_id, pad_to_seq_len=True)
    offline: List[Dict] = []  # members of the offline pack being collected (samples carrying pack_id / pack_size)

    def batches(packs):
        for p in packs:
            b = {"tokens": p["tokens"][None], "labels": p["labels"][None], "loss_mask": p["loss_mask"][None],
                 "position_ids": p["position_ids"].unsqueeze(1), "cu_seqlens": p["cu_seqlens"],
                 "pixels": p["pixels"].float(), "grid_thw": p["grid_thw"]}
            if pin_memory:
                b = {k: v.pin_memory() for k, v in b.items()}
            b["num_valid_tokens"] = int(p["loss_mask"].sum().item())
            yield b

    for raw in samples:
        enc = encoder.encode(raw)
        if enc is None:
            continue  # gated by the task encoder (over-long sample)
        if "mrope" not in enc:  # family encoders (data/task_encoders.py) bring their own position ids
            enc["mrope"] = mrope_ids(enc["tokens"], enc["grid_thw"], encoder.img_id, merge_size)
        enc = merge_video_into_image_stream(enc, encoder.img_id, getattr(getattr(encoder, "sp", None), "video", None))
        if "pack_id" in raw:
            # packs were decided offline: the members of a pack arrive consecutively and form one row as they are
            # (the offline lengths are estimates: a pack that comes out too long sheds its last members)
            offline.append(enc)
            if len(offline) >= int(raw["pack_size"]):
                while sum(e["tokens"].numel() for e in offline) > seq_len and len(offline) > 1:
                    offline.pop()
                if offline[0]["tokens"].numel() <= seq_len:
                    yield from batches([packer._pack(offline)])
                offline = []
            continue
        yield from batches(packer.add(enc))
    yield from batches(packer.flush())
