"""Per-family multimodal task encoders: raw sample -> model inputs, one class per model family because the families
differ in how an image becomes tokens (reference: loongforge/data/multimodal/{vlm,kimi,llava_ov,minicpm_v_4_6,ernie}
_task_encoder.py, loongforge/data/multimodal/internvl/).

A raw sample is one of
  * captioning: ``{"image": arr, "caption": str}``
  * VQA:        ``{"image": arr | "images": [arr], "context": str, "answer": str}`` (context carries the markers)
  * chat:       ``{"images": [arr], "videos": [[frame arrs]], "conversation": [{"role", "content"}]}``
Every encoder returns the dict the online packer and the vision-language trainer consume: ``tokens``, ``labels``
(next-token targets), ``loss_mask``, ``pixels`` + ``grid_thw`` (or ``pixel_tiles`` for tile-based encoders), and
``mrope`` position ids ``[3, T]``; family extras (``token_type``) ride along.

| family     | image -> tokens                                                                                   |
|------------|---------------------------------------------------------------------------------------------------|
| qwen2_vl / qwen2_5_vl / qwen3_vl | native resolution, (h/p/m)(w/p/m) tokens between vision start / end markers; video = frames grouped by the temporal patch (Qwen3-VL: one time-stamped block per frame group) |
| internvl   | dynamic tiling into up to `max_tiles` 448 x 448 tiles (+ thumbnail), 256 context tokens per tile  |
| llava_ov   | native resolution RICE-ViT patches, merged 2 x 2, plain ``<image>`` expansion, no wrappers         |
| kimi_vl    | native resolution, tokens = (h/mh)(w/mw) (time pooled away), media begin / end wrappers, over-long samples gated |
| minicpm_v  | sides rounded to multiples of 28, video frame counts to multiples of 2, 4 x downsampling of the merged grid |
| ernie_vl   | like qwen, plus token types (text / image experts) and (t, h, w) positions in which an image takes one time step |
"""
from __future__ import annotations

import dataclasses
import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .multimodal import IGNORE, VisionPreprocess
from .position_ids import internvl_ids, mrope_ids, qwen2_5_vl_ids, qwen3_vl_ids

IMAGE_MARKER, VIDEO_MARKER = "<image>", "<video>"


@dataclasses.dataclass
class SpecialTokens:
    """Token ids the encoders insert. `image` / `video` are the placeholder ids the model replaces by embeddings."""
    image: int
    video: Optional[int] = None
    vision_start: Optional[int] = None
    vision_end: Optional[int] = None
    eos: Optional[int] = None


def to_conversation(sample: Dict) -> Tuple[List[Dict[str, str]], List[np.ndarray], List[List[np.ndarray]]]:
    """Normalises the three raw sample kinds to (conversation, images, videos)."""
    if "conversation" in sample:
        return list(sample["conversation"]), list(sample.get("images", [])), list(sample.get("videos", []))
    images = list(sample.get("images", [])) or ([sample["image"]] if sample.get("image") is not None else [])
    if "caption" in sample:
        return ([{"role": "user", "content": IMAGE_MARKER * len(images)},
                 {"role": "assistant", "content": sample["caption"]}], images, [])
    ctx = sample["context"]
    if IMAGE_MARKER not in ctx:
        ctx = IMAGE_MARKER * len(images) + ctx
    return [{"role": "user", "content": ctx}, {"role": "assistant", "content": sample["answer"]}], images, []


class TaskEncoder:
    """Shared turn walker: splits every turn at the media markers, lets the family hooks turn each medium into token
    ids and pixel data, masks everything outside assistant turns."""

    family = "base"

    def __init__(self, tokenize: Callable[[str], List[int]], special: SpecialTokens,
                 vision: Optional[VisionPreprocess] = None, max_length: Optional[int] = None,
                 overlong: str = "drop", roles: Tuple[str, str] = ("user", "assistant"),
                 turn_prefix: Optional[Callable[[str], str]] = None, turn_suffix: str = ""):
        self.tok, self.sp, self.vision = tokenize, special, vision or VisionPreprocess()
        self.max_length, self.overlong, self.roles = max_length, overlong, roles
        self.turn_prefix, self.turn_suffix = turn_prefix, turn_suffix
        self.img_id = special.image  # what `vlm_batch_iterator` reads

    # ---- family hooks
    def encode_image(self, image: np.ndarray, acc: Dict) -> List[int]:
        p, g = self.vision(image)
        acc["pixels"].append(p)
        acc["grids"].append(g)
        n = p.shape[0] // self.vision.merge_size ** 2
        return self.wrap([self.sp.image] * n)

    def encode_video(self, frames: Sequence[np.ndarray], acc: Dict) -> List[int]:
        """Frames are grouped by the temporal patch; one grid (t, h, w) for the whole clip."""
        tp = self.vision.temporal_patch_size
        frames = list(frames) + [frames[-1]] * (-len(frames) % tp)
        pats = []
        for i in range(0, len(frames), tp):
            per = [self.vision(f)[0].reshape(-1, 3, tp, self.vision.patch_size, self.vision.patch_size)[:, :, 0]
                   for f in frames[i:i + tp]]
            pats.append(np.stack(per, 2).reshape(per[0].shape[0], -1))
        _, gh, gw = self.vision(frames[0])[1]
        acc["vpixels"].append(np.concatenate(pats))
        acc["vgrids"].append((len(frames) // tp, gh, gw))
        n = (len(frames) // tp) * (gh // self.vision.merge_size) * (gw // self.vision.merge_size)
        vid = self.sp.video if self.sp.video is not None else self.sp.image
        return self.wrap([vid] * n)

    def wrap(self, ids: List[int]) -> List[int]:
        s, e = self.sp.vision_start, self.sp.vision_end
        return ([s] if s is not None else []) + ids + ([e] if e is not None else [])

    def positions(self, tokens: torch.Tensor, grids, vgrids) -> torch.Tensor:
        return mrope_ids(tokens, grids, self.sp.image, self.vision.merge_size, vgrids, self.sp.video)

    def finish(self, out: Dict, acc: Dict) -> Dict:
        return out

    # ---- the walker
    def encode(self, sample: Dict) -> Optional[Dict[str, torch.Tensor]]:
        conv, images, videos = to_conversation(sample)
        acc = {"pixels": [], "grids": [], "vpixels": [], "vgrids": [], "tiles": [], "order": []}
        ids: List[int] = []
        labels: List[int] = []
        ki = kv = 0
        for turn in conv:
            text = (self.turn_prefix(turn["role"]) if self.turn_prefix else "") + turn["content"] + self.turn_suffix
            t_ids: List[int] = []
            rest = text
            while rest:
                i_img, i_vid = rest.find(IMAGE_MARKER), rest.find(VIDEO_MARKER)
                cands = [(i, m) for i, m in ((i_img, IMAGE_MARKER), (i_vid, VIDEO_MARKER)) if i >= 0]
                if not cands:
                    t_ids += self.tok(rest)
                    break
                i, m = min(cands)
                if i:
                    t_ids += self.tok(rest[:i])
                if m == IMAGE_MARKER:
                    if ki >= len(images):
                        raise ValueError("more <image> markers than images")
                    t_ids += self.encode_image(images[ki], acc)
                    acc["order"].append(0)
                    ki += 1
                else:
                    if kv >= len(videos):
                        raise ValueError("more <video> markers than videos")
                    t_ids += self.encode_video(videos[kv], acc)
                    acc["order"].append(1)
                    kv += 1
                rest = rest[i + len(m):]
            if turn["role"] == self.roles[1]:
                if self.sp.eos is not None:
                    t_ids.append(self.sp.eos)
                labels += t_ids
            else:
                labels += [IGNORE] * len(t_ids)
            ids += t_ids
        if ki != len(images) or kv != len(videos):
            raise ValueError(f"{len(images)} images / {len(videos)} videos but {ki} / {kv} markers")
        if self.max_length is not None and len(ids) > self.max_length:
            if self.overlong == "drop":
                return None
            # truncation may not cut through a medium: keep whole media only
            cut = self.max_length
            media = {self.sp.image, self.sp.video}
            while cut > 0 and (ids[cut - 1] in media or (cut < len(ids) and ids[cut] in media)):
                cut -= 1
            if any(t in media for t in ids[cut:]):
                return None  # media would be lost: pixel data and tokens would disagree
            ids, labels = ids[:cut], labels[:cut]
        media_ids = {x for x in (self.sp.image, self.sp.video, self.sp.vision_start, self.sp.vision_end) if x is not None}
        labels = [IGNORE if t in media_ids else l for t, l in zip(ids, labels)]  # never predict placeholders
        tokens = torch.tensor(ids, dtype=torch.long)
        lab = torch.tensor(labels[1:] + [IGNORE], dtype=torch.long)
        grids = torch.tensor(acc["grids"], dtype=torch.long).view(-1, 3)
        vgrids = torch.tensor(acc["vgrids"], dtype=torch.long).view(-1, 3)
        out = {"tokens": tokens, "labels": lab.clamp(min=0), "loss_mask": (lab != IGNORE).float(),
               "pixels": torch.from_numpy(np.concatenate(acc["pixels"])) if acc["pixels"] else torch.zeros(0, 0),
               "grid_thw": grids}
        if acc["vpixels"]:
            out["video_pixels"] = torch.from_numpy(np.concatenate(acc["vpixels"]))
            out["video_grid_thw"] = vgrids
            out["media_order"] = torch.tensor(acc["order"], dtype=torch.long)   # 0 image / 1 video, in token order
        if len(vgrids) and self.sp.video is None:
            # no video placeholder of its own: videos are written with the image placeholder, so the position function
            # walks ONE grid list in token order
            ig, vg = iter(grids), iter(vgrids)
            merged = torch.stack([next(ig) if kind == 0 else next(vg) for kind in acc["order"]])
            out["mrope"] = self.positions(tokens, merged, None)
        else:
            out["mrope"] = self.positions(tokens, grids if len(grids) else None, vgrids if len(vgrids) else None)
        return self.finish(out, acc)


class Qwen2VLTaskEncoder(TaskEncoder):
    family = "qwen2_vl"


class Qwen25VLTaskEncoder(TaskEncoder):
    """Temporal positions follow real time: `second_per_grid_t` = temporal patch / fps."""
    family = "qwen2_5_vl"

    def __init__(self, *a, fps: float = 2.0, tokens_per_second: float = 2.0, **kw):
        super().__init__(*a, **kw)
        self.fps, self.tps = fps, tokens_per_second

    def positions(self, tokens, grids, vgrids):
        sec = [self.vision.temporal_patch_size / self.fps] * (0 if vgrids is None else len(vgrids))
        return qwen2_5_vl_ids(tokens, grids, self.sp.image, self.vision.merge_size, vgrids, self.sp.video, sec, self.tps)


class Qwen3VLTaskEncoder(TaskEncoder):
    """Videos become one block per frame group, each preceded by its time stamp as text (``<1.5 seconds>``)."""
    family = "qwen3_vl"

    def __init__(self, *a, fps: float = 2.0, **kw):
        super().__init__(*a, **kw)
        self.fps = fps

    def encode_video(self, frames, acc):
        before = len(acc["vgrids"])
        flat = super().encode_video(frames, acc)
        t, gh, gw = acc["vgrids"][before]
        per = (gh // self.vision.merge_size) * (gw // self.vision.merge_size)
        vid = self.sp.video if self.sp.video is not None else self.sp.image
        out: List[int] = []
        for g in range(t):
            stamp = (g * self.vision.temporal_patch_size + (self.vision.temporal_patch_size - 1) / 2) / self.fps
            out += self.tok(f"<{stamp:.1f} seconds>") + self.wrap([vid] * per)
        assert sum(1 for x in out if x == vid) == sum(1 for x in flat if x == vid)
        return out

    def positions(self, tokens, grids, vgrids):
        return qwen3_vl_ids(tokens, grids, self.sp.image, self.vision.merge_size, vgrids, self.sp.video)


class InternVLTaskEncoder(TaskEncoder):
    """Tile-based: pixels are ``pixel_tiles`` [n, 3, 448, 448]; positions are the token-type based InternVL ids."""
    family = "internvl"

    def __init__(self, *a, tile: int = 448, max_tiles: int = 12, tokens_per_tile: int = 256, use_thumbnail: bool = True,
                 mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225), **kw):
        super().__init__(*a, **kw)
        self.tile, self.max_tiles, self.per_tile, self.thumb = tile, max_tiles, tokens_per_tile, use_thumbnail
        self.mean, self.std = np.asarray(mean, np.float32), np.asarray(std, np.float32)

    def _resize(self, image: np.ndarray, h: int, w: int) -> np.ndarray:
        H, W = image.shape[:2]
        ys, xs = (np.arange(h) * H / h).astype(int), (np.arange(w) * W / w).astype(int)
        x = image[ys][:, xs].astype(np.float32) / 255.0
        return ((x - self.mean) / self.std).transpose(2, 0, 1)

    def encode_image(self, image, acc):
        from ..runtime.sft_families import internvl_tile_grid
        H, W = image.shape[:2]
        c, r = internvl_tile_grid(W, H, max_tiles=self.max_tiles, tile=self.tile)
        big = self._resize(image, r * self.tile, c * self.tile)
        tiles = [big[:, i * self.tile:(i + 1) * self.tile, j * self.tile:(j + 1) * self.tile]
                 for i in range(r) for j in range(c)]
        if self.thumb and len(tiles) > 1:
            tiles.append(self._resize(image, self.tile, self.tile))
        acc["tiles"].append(np.stack(tiles))
        return self.wrap([self.sp.image] * (len(tiles) * self.per_tile))

    def encode_video(self, frames, acc):
        out: List[int] = []
        for k, f in enumerate(frames):  # every frame is one tile, announced as text
            acc["tiles"].append(self._resize(f, self.tile, self.tile)[None])
            out += self.tok(f"Frame{k + 1}: ") + self.wrap([self.sp.image] * self.per_tile)
        return out

    def positions(self, tokens, grids, vgrids):
        media = {x for x in (self.sp.image, self.sp.vision_start, self.sp.vision_end) if x is not None}
        types = torch.tensor([1 if t in media else 0 for t in tokens.tolist()])
        return internvl_ids(types).unsqueeze(0).expand(3, -1).contiguous()

    def finish(self, out, acc):
        tiles = np.concatenate(acc["tiles"]) if acc["tiles"] else np.zeros((0, 3, self.tile, self.tile), np.float32)
        out["pixel_tiles"] = torch.from_numpy(tiles)
        out["image_flags"] = torch.ones(tiles.shape[0], dtype=torch.long)
        return out


class LlavaOVTaskEncoder(TaskEncoder):
    """LLaVA-OneVision-1.5: plain placeholder expansion, no begin / end wrappers."""
    family = "llava_ov"

    def wrap(self, ids):
        return ids


class KimiVLTaskEncoder(TaskEncoder):
    """Kimi-VL / K2.5: time is pooled away inside the projector, so a clip of t frame groups still costs
    (h / mh)(w / mw) tokens; samples longer than `max_length` are gated (dropped or cut at a media boundary)."""
    family = "kimi_vl"

    def __init__(self, *a, merge_kernel: Tuple[int, int] = (2, 2), **kw):
        kw.setdefault("overlong", "truncate")
        super().__init__(*a, **kw)
        self.merge_kernel = merge_kernel

    def encode_image(self, image, acc):
        p, g = self.vision(image)
        acc["pixels"].append(p)
        acc["grids"].append(g)
        return self.wrap([self.sp.image] * ((g[1] // self.merge_kernel[0]) * (g[2] // self.merge_kernel[1])))

    def encode_video(self, frames, acc):
        before = len(acc["vgrids"])
        super().encode_video(frames, acc)
        _, gh, gw = acc["vgrids"][before]
        vid = self.sp.video if self.sp.video is not None else self.sp.image
        return self.wrap([vid] * ((gh // self.merge_kernel[0]) * (gw // self.merge_kernel[1])))

    def positions(self, tokens, grids, vgrids):
        # one text-like position per token: Kimi's language model uses ordinary rotary positions
        return torch.arange(tokens.numel()).unsqueeze(0).expand(3, -1).contiguous()


class MiniCPMVTaskEncoder(TaskEncoder):
    """MiniCPM-V 4.6: sides rounded to multiples of 28 within a pixel budget, frame counts to multiples of 2, and the
    merged grid is downsampled 2 x 2 once more by the projector."""
    family = "minicpm_v"

    def __init__(self, *a, size_factor: int = 28, frame_factor: int = 2, downsample: int = 2, **kw):
        super().__init__(*a, **kw)
        self.size_factor, self.frame_factor, self.down = size_factor, frame_factor, downsample

    def _tokens(self, gh: int, gw: int, t: int = 1) -> int:
        m = self.vision.merge_size * self.down
        return t * math.ceil(gh / m) * math.ceil(gw / m)

    def encode_image(self, image, acc):
        p, g = self.vision(image)
        acc["pixels"].append(p)
        acc["grids"].append(g)
        return self.wrap([self.sp.image] * self._tokens(g[1], g[2]))

    def encode_video(self, frames, acc):
        frames = list(frames) + [frames[-1]] * (-len(frames) % self.frame_factor)
        before = len(acc["vgrids"])
        super().encode_video(frames, acc)
        t, gh, gw = acc["vgrids"][before]
        vid = self.sp.video if self.sp.video is not None else self.sp.image
        return self.wrap([vid] * self._tokens(gh, gw, t))

    def positions(self, tokens, grids, vgrids):
        return torch.arange(tokens.numel()).unsqueeze(0).expand(3, -1).contiguous()


class ErnieVLTaskEncoder(TaskEncoder):
    """ERNIE-4.5-VL: token types route tokens to the text / vision experts; an image takes ONE time step with
    (row, column) offsets and the text after it continues from the largest index used so far."""
    family = "ernie_vl"

    def positions(self, tokens, grids, vgrids):
        from ..runtime.sft_families import ernie_token_types_and_positions
        m = self.vision.merge_size
        hw = [(g[1] // m, g[2] // m) for g in (grids.tolist() if grids is not None else [])]
        self._types, pos = ernie_token_types_and_positions(tokens, self.sp.image, hw)
        return pos

    def finish(self, out, acc):
        out["token_type"] = self._types
        return out


TASK_ENCODERS = {c.family: c for c in (Qwen2VLTaskEncoder, Qwen25VLTaskEncoder, Qwen3VLTaskEncoder, InternVLTaskEncoder,
                                       LlavaOVTaskEncoder, KimiVLTaskEncoder, MiniCPMVTaskEncoder, ErnieVLTaskEncoder)}
# aliases: names used by model configurations and vision families
TASK_ENCODERS.update({"qwen2_5_vit": Qwen25VLTaskEncoder, "qwen2_vit": Qwen2VLTaskEncoder, "qwen3_vl_vit": Qwen3VLTaskEncoder,
                      "qwen3_5": Qwen3VLTaskEncoder, "intern_vit": InternVLTaskEncoder, "rice_vit": LlavaOVTaskEncoder,
                      "moon_vit": KimiVLTaskEncoder, "minicpm_v_vit": MiniCPMVTaskEncoder, "ernie_vit": ErnieVLTaskEncoder,
                      "ernie4_5_vl": ErnieVLTaskEncoder})


def build_task_encoder(family: str, tokenize, special: SpecialTokens, vision: Optional[VisionPreprocess] = None,
                       **kw) -> TaskEncoder:
    cls = TASK_ENCODERS.get(family)
    if cls is None:
        raise KeyError(f"no task encoder for family {family!r}; known: {sorted(TASK_ENCODERS)}")
    return cls(tokenize, special, vision, **kw)
