"""Family-specific SFT batch construction for InternVL and ERNIE-4.5-VL (reference:
loongforge/train/sft/sft_internvl.py:48-249, loongforge/train/sft/sft_ernie.py:37-257).

* InternVL: each image is cut into up to `max_tiles` 448x448 tiles on the grid whose aspect ratio is closest to the
  image's (plus a thumbnail when more than one tile); every tile contributes ``(448 / 14)^2 / 4 = 256`` context tokens
  written as ``<img>`` + ``<IMG_CONTEXT>`` * n + ``</img>``.
* ERNIE-4.5-VL: tokens carry a modality type (0 text, 1 image) that routes them to the text / vision experts, and 3-D
  position ids: text advances all three axes together; an image occupies one time step with (row, column) offsets, and
  the text after it continues from the largest index used so far.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch


# ---- InternVL ---------------------------------------------------------------------------------------------------------
def internvl_tile_grid(width: int, height: int, min_tiles: int = 1, max_tiles: int = 12, tile: int = 448) -> Tuple[int, int]:
    """(columns, rows) of the tiling whose aspect ratio is closest to the image's; ties prefer more tiles when the image
    is large enough to fill them."""
    ratio = width / height
    cands = sorted({(i, j) for n in range(min_tiles, max_tiles + 1) for i in range(1, n + 1) for j in range(1, n + 1)
                    if min_tiles <= i * j <= max_tiles}, key=lambda x: x[0] * x[1])
    best, best_diff = (1, 1), float("inf")
    area = width * height
    for c, r in cands:
        diff = abs(ratio - c / r)
        if diff < best_diff:
            best, best_diff = (c, r), diff
        elif diff == best_diff and area > 0.5 * tile * tile * c * r:
            best = (c, r)
    return best


def internvl_num_tiles(width: int, height: int, max_tiles: int = 12, use_thumbnail: bool = True) -> int:
    c, r = internvl_tile_grid(width, height, max_tiles=max_tiles)
    n = c * r
    return n + 1 if (use_thumbnail and n > 1) else n


def internvl_expand_image_tokens(token_ids: Sequence[int], image_sizes: Sequence[Tuple[int, int]], *, image_marker_id: int,
                                 img_start_id: int, img_context_id: int, img_end_id: int, tokens_per_tile: int = 256,
                                 max_tiles: int = 12) -> Tuple[List[int], List[int]]:
    """Replaces each marker by ``<img> ctx*n </img>``. Returns (ids, tiles per image)."""
    out: List[int] = []
    tiles: List[int] = []
    k = 0
    for t in token_ids:
        if t == image_marker_id:
            n = internvl_num_tiles(*image_sizes[k], max_tiles=max_tiles)
            tiles.append(n)
            out += [img_start_id] + [img_context_id] * (n * tokens_per_tile) + [img_end_id]
            k += 1
        else:
            out.append(t)
    if k != len(image_sizes):
        raise ValueError(f"{len(image_sizes)} images but {k} markers")
    return out, tiles


def internvl_batch(samples: List[Dict], pad_id: int = 0) -> Dict[str, torch.Tensor]:
    """samples: ``{"input_ids", "labels" (-100 = masked), "pixel_tiles" [n_tiles, 3, 448, 448]}`` -> packed batch."""
    ids = torch.cat([torch.as_tensor(s["input_ids"]) for s in samples])
    lab = torch.cat([torch.as_tensor(s["labels"][1:] + [-100]) for s in samples])
    lens = [len(s["input_ids"]) for s in samples]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    tiles = [s["pixel_tiles"] for s in samples if s.get("pixel_tiles") is not None and len(s["pixel_tiles"])]
    return {"tokens": ids, "labels": lab.clamp(min=0), "loss_mask": (lab != -100).float(),
            "position_ids": torch.cat([torch.arange(n) for n in lens]), "cu_seqlens": cu,
            "pixel_tiles": torch.cat(tiles) if tiles else torch.zeros(0, 3, 448, 448),
            "image_flags": torch.ones(sum(t.shape[0] for t in tiles), dtype=torch.long)}


# ---- ERNIE-4.5-VL -----------------------------------------------------------------------------------------------------
def ernie_token_types_and_positions(token_ids: torch.Tensor, image_token_id: int, grids_hw: Sequence[Tuple[int, int]]
                                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (token_type [T] 0/1, position_ids [3, T] as (t, h, w)). `grids_hw`: merged-token grid of every image, in order;
    each run of image tokens must have h * w tokens."""
    T = token_ids.numel()
    tt = (token_ids == image_token_id).long()
    pos = torch.zeros(3, T, dtype=torch.long)
    cur, i, k = 0, 0, 0
    ids = token_ids.tolist()
    while i < T:
        if ids[i] != image_token_id:
            pos[:, i] = cur
            cur += 1
            i += 1
            continue
        h, w = grids_hw[k]
        k += 1
        n = h * w
        if ids[i:i + n] != [image_token_id] * n:
            raise ValueError("run of image tokens shorter than its grid")
        rows = torch.arange(h).repeat_interleave(w)
        cols = torch.arange(w).repeat(h)
        pos[0, i:i + n] = cur
        pos[1, i:i + n] = cur + rows
        pos[2, i:i + n] = cur + cols
        cur += max(h, w)
        i += n
    return tt, pos


def ernie_forward_kwargs(batch: Dict[str, torch.Tensor], image_token_id: int) -> Dict[str, torch.Tensor]:
    """Extra model inputs for an ERNIE batch: modality types for the expert routing and 3-D positions for the rotary."""
    tt, pos = ernie_token_types_and_positions(batch["tokens"].reshape(-1).cpu(), image_token_id,
                                              [tuple(g) for g in batch["merged_grids"]])
    dev = batch["tokens"].device
    return {"token_type": tt.to(dev), "position_ids": pos.to(dev)}
