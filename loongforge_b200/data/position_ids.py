"""Position-id functions: plain text positions and the multimodal (M-RoPE) index of Qwen2-VL style
models (loongforge/train/get_position_idx_func.py:10-348). ``mrope_ids`` returns ``[3, T]`` (t, h, w
streams): text tokens advance all three streams together; the tokens of an image take the position
of their merged patch inside the image grid, offset by the running maximum."""
from __future__ import annotations

from typing import List, Optional

import torch


def text_position_ids(seq_len: int, batch: int = 1, device=None) -> torch.Tensor:
    return torch.arange(seq_len, device=device).unsqueeze(0).expand(batch, -1).contiguous()


def packed_position_ids(cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Positions restarting at every packed-sequence boundary."""
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    return torch.cat([torch.arange(n, device=cu_seqlens.device) for n in lens])


def mrope_ids(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], image_token_id: int,
              spatial_merge_size: int = 2, video_grid_thw: Optional[torch.Tensor] = None,
              video_token_id: Optional[int] = None) -> torch.Tensor:
    """input_ids [T] (one sample) -> position ids [3, T]."""
    T = input_ids.numel()
    ids = input_ids.tolist()
    grids: List[List[int]] = image_grid_thw.tolist() if image_grid_thw is not None else []
    vgrids: List[List[int]] = video_grid_thw.tolist() if video_grid_thw is not None else []
    pos = torch.zeros(3, T, dtype=torch.long)
    i, nxt, gi, vi = 0, 0, 0, 0
    while i < T:
        tok = ids[i]
        is_img = tok == image_token_id
        is_vid = video_token_id is not None and tok == video_token_id
        if not (is_img or is_vid):
            pos[:, i] = nxt
            nxt += 1
            i += 1
            continue
        t, h, w = (grids[gi] if is_img else vgrids[vi])
        if is_img:
            gi += 1
        else:
            vi += 1
        gh, gw = h // spatial_merge_size, w // spatial_merge_size
        n = t * gh * gw
        tt = torch.arange(t).view(-1, 1, 1).expand(t, gh, gw).flatten()
        hh = torch.arange(gh).view(1, -1, 1).expand(t, gh, gw).flatten()
        ww = torch.arange(gw).view(1, 1, -1).expand(t, gh, gw).flatten()
        n = min(n, T - i)
        pos[0, i:i + n] = tt[:n] + nxt
        pos[1, i:i + n] = hh[:n] + nxt
        pos[2, i:i + n] = ww[:n] + nxt
        nxt = int(pos[:, i:i + n].max()) + 1
        i += n
    return pos.to(input_ids.device)
