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


def qwen2_5_vl_ids(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], image_token_id: int,
                   spatial_merge_size: int = 2, video_grid_thw: Optional[torch.Tensor] = None,
                   video_token_id: Optional[int] = None, second_per_grid_ts: Optional[List[float]] = None,
                   tokens_per_second: float = 2.0) -> torch.Tensor:
    """Qwen2.5-VL: like `mrope_ids`, but the temporal index of video frame group g is
    ``floor(g * second_per_grid_t * tokens_per_second)``: frames further apart in time sit further apart in the t stream
    (reference: loongforge/train/get_position_idx_func.py:181-338)."""
    pos = mrope_ids(input_ids, image_grid_thw, image_token_id, spatial_merge_size, video_grid_thw, video_token_id)
    if video_grid_thw is None or video_token_id is None or not second_per_grid_ts:
        return pos
    ids = input_ids.tolist()
    T, i, vi, shift = len(ids), 0, 0, 0
    pos = pos.clone()
    vg = video_grid_thw.tolist()
    while i < T:
        if ids[i] != video_token_id:
            pos[:, i] += shift
            i += 1
            continue
        t, h, w = vg[vi]
        per = (h // spatial_merge_size) * (w // spatial_merge_size)
        n = min(t * per, T - i)
        base = int(pos[0, i]) + shift
        sec = float(second_per_grid_ts[vi]) if vi < len(second_per_grid_ts) else 1.0
        tt = (torch.arange(t, dtype=torch.float64) * sec * tokens_per_second).floor().long().repeat_interleave(per)[:n]
        old_max = int(pos[:, i:i + n].max()) + shift
        pos[1:, i:i + n] += shift
        pos[0, i:i + n] = base + tt
        shift += max(int(pos[:, i:i + n].max()) - old_max, 0)
        vi += 1
        i += n
    return pos


def qwen3_vl_ids(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], image_token_id: int,
                 spatial_merge_size: int = 2, video_grid_thw: Optional[torch.Tensor] = None,
                 video_token_id: Optional[int] = None) -> torch.Tensor:
    """Qwen3-VL / Qwen3.5: videos are written frame by frame with a text time stamp before each frame
    (``<t1> <vision_start> frame <vision_end> <t2> ...``), so a video grid (t, h, w) is t grids (1, h, w) and time is
    carried by the stamps, not by the t stream (reference: loongforge/train/get_position_idx_func.py:10-148)."""
    if video_grid_thw is not None and video_grid_thw.numel():
        v = torch.repeat_interleave(video_grid_thw, video_grid_thw[:, 0], dim=0).clone()
        v[:, 0] = 1
        video_grid_thw = v
    return mrope_ids(input_ids, image_grid_thw, image_token_id, spatial_merge_size, video_grid_thw, video_token_id)


def internvl_ids(token_types: torch.Tensor, vision_type: int = 1, language_type: int = 0) -> torch.Tensor:
    """InternVL: `token_types` [T] marks vision tokens. The first and last token of every vision run (begin / end of
    image) count as language; language tokens and the first inner vision token after language advance the position,
    the other inner vision tokens share it (reference: loongforge/train/get_position_idx_func.py:151-178)."""
    x = token_types.clone()
    vis = x == vision_type
    lang = x == language_type
    edge = torch.zeros_like(vis)
    edge[1:] |= vis[1:] & lang[:-1]
    edge[0] |= vis[0]
    edge[:-1] |= vis[:-1] & lang[1:]
    edge[-1] |= vis[-1]
    x[edge] = language_type
    lang, vis = x == language_type, x == vision_type
    step = torch.zeros_like(x, dtype=torch.long)
    step[1:] = (lang[1:] | (vis[1:] & lang[:-1])).long()
    return step.cumsum(0)


POSITION_ID_FUNCS = {"text": text_position_ids, "packed": packed_position_ids, "qwen2_vl": mrope_ids,
                     "qwen2_5_vl": qwen2_5_vl_ids, "qwen3_vl": qwen3_vl_ids, "internvl": internvl_ids}


def get_position_id_func(name: str):
    """Position-id function by the name the model configuration selects (YAML resolver ``${position_func:...}``)."""
    if name not in POSITION_ID_FUNCS:
        raise KeyError(f"unknown position-id function {name!r}; known: {sorted(POSITION_ID_FUNCS)}")
    return POSITION_ID_FUNCS[name]
