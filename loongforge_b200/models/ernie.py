"""ERNIE-4.5-VL specifics: modality-routed expert sets and the 3-D rotary layout.

* ``MultiTypeMoELayer``: text tokens go through the text experts (own router), vision tokens through the
  vision experts (own router, usually a smaller FFN); a shared expert sees every token
  (loongforge/models/foundation/ernie4_5_vl/ernie_moe_layer.py:59-322, ernie_experts.py:63-340,
  ernie_router.py:142-200).
* ``ernie_3d_angles``: of the D/2 rotary frequencies the LAST ``freq_allocation`` follow the temporal
  position; in the rest even-indexed frequencies follow the height position and odd-indexed ones the
  width position; pairs are rotated in the interleaved (x0, x1), (x2, x3), ... layout
  (loongforge/models/foundation/ernie4_5_vl/ernie_pos_embedding.py:12-180).
"""
from __future__ import annotations

import copy
from typing import Optional

import torch
import torch.nn as nn

from ..parallel import state as ps
from .config import TransformerConfig
from .moe import MoELayer
from .transformer import RotaryInputs


def ernie_3d_angles(position_ids: torch.Tensor, rot_dim: int, base: float, freq_allocation: int) -> RotaryInputs:
    """position_ids [3, T] as (t, h, w) -> angles [T, rot_dim/2] for an INTERLEAVED rotation."""
    half = rot_dim // 2
    inv = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=position_ids.device) / rot_dim))
    j = torch.arange(half, device=position_ids.device)
    stream = torch.where(j >= half - freq_allocation, torch.zeros_like(j), 1 + (j % 2))  # 0 = t, 1 = h, 2 = w
    pos = position_ids.float()[stream, :].t()  # [T, half]
    return RotaryInputs(freqs=(pos * inv).contiguous())


class MultiTypeMoELayer(nn.Module):
    """Two expert sets selected by ``token_type`` (0 = text, 1 = vision)."""

    def __init__(self, cfg: TransformerConfig, key: str, layer_number: int, *, device=None, parallel_state=None):
        super().__init__()
        text_cfg = copy.copy(cfg)
        text_cfg.moe_shared_expert_intermediate_size = None
        vis_cfg = copy.copy(text_cfg)
        vis_cfg.num_moe_experts = cfg.moe_vision_num_experts or cfg.num_moe_experts
        vis_cfg.moe_ffn_hidden_size = cfg.moe_vision_ffn_hidden_size or cfg.moe_ffn_hidden_size
        self.text = MoELayer(text_cfg, key + ".text_moe", layer_number, device=device, parallel_state=parallel_state)
        self.vision = MoELayer(vis_cfg, key + ".vision_moe", layer_number, device=device, parallel_state=parallel_state)
        if cfg.moe_shared_expert_intermediate_size:
            from .transformer import MLP
            self.shared_experts = MLP(cfg, key + ".shared_experts", ffn_hidden=cfg.moe_shared_expert_intermediate_size,
                                      fused_norm=False, device=device, parallel_state=parallel_state,
                                      sequence_parallel=False)
        else:
            self.shared_experts = None
        self.token_type: Optional[torch.Tensor] = None  # [T] set per micro-batch by the model wrapper
        self.cfg, self.state_name = cfg, parallel_state

    def set_token_type(self, token_type: Optional[torch.Tensor]):
        self.token_type = token_type

    def forward(self, x: torch.Tensor, seq_lens=None) -> torch.Tensor:
        from ..parallel import mappings as M

        st = ps.get_state(self.state_name)
        sp = self.cfg.sequence_parallel and st.dims.tp > 1
        tt = self.token_type
        if tt is not None and sp and tt.numel() == x.shape[0] * st.dims.tp:
            tt = tt[st.tp_rank * x.shape[0]:(st.tp_rank + 1) * x.shape[0]]  # this rank's sequence shard
        if tt is None:
            out = self.text(x, seq_lens)
        else:
            vis = tt.bool()
            out = torch.zeros_like(x)
            # both branches always run (possibly on zero tokens) so that every rank issues the same collectives
            ti, vi = (~vis).nonzero(as_tuple=True)[0], vis.nonzero(as_tuple=True)[0]
            out = out.index_add(0, ti, self.text(x.index_select(0, ti)))
            out = out.index_add(0, vi, self.vision(x.index_select(0, vi)))
        if self.shared_experts is not None:
            if sp:
                # the shared expert is tensor parallel over the WHOLE token set of the TP group
                g = st.group("tp")
                ys = self.shared_experts(M.gather_from_sequence_parallel_region(x, g, False))
                out = out + M.scatter_to_sequence_parallel_region(ys, g)
            else:
                out = out + self.shared_experts(x)
        return out
