"""Manifold-constrained hyper-connections (DeepSeek-V4): ``n`` parallel residual streams per token.

For a sub-layer ``F`` and streams ``X [n, C]`` of one token::

    h      = H_pre  X                       (1 x n  read weights,   sigmoid)
    X_next = H_res  X + H_post^T F(h)       (n x n  stream mixing,  doubly stochastic by Sinkhorn;
                                             n x 1  write weights,  2 * sigmoid)

All three maps are token-dependent: a static base plus a small learned gate times a linear read-out of
the RMS-normalised flattened streams. ``HyperHead`` folds the streams back into one vector before
the final norm. Reference: the TransformerBlock hook at
loongforge/models/foundation/language_transformer_block.py:92-105 and the ``hc_*`` fields of
loongforge/models/foundation/deepseek_v4/deepseek_v4_config.py:54-56,86-89.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..parallel import layers as PL


def sinkhorn(logits: torch.Tensor, iters: int) -> torch.Tensor:
    """Rows and columns of exp(logits) [..., n, n] alternately normalised `iters` times."""
    m = torch.exp(logits - logits.amax(dim=(-1, -2), keepdim=True))
    for _ in range(iters):
        m = m / m.sum(-1, keepdim=True)
        m = m / m.sum(-2, keepdim=True)
    return m


class HyperConnection(nn.Module):
    def __init__(self, hidden: int, n: int, sinkhorn_iters: int, gate_init: float, eps: float, key: str, device=None,
                 sequence_parallel: bool = False):
        super().__init__()
        self.n, self.hidden, self.iters, self.eps = n, hidden, sinkhorn_iters, eps
        width = 2 * n + n * n
        self.fn = nn.Parameter(PL.init_full_then_slice(key + ".fn", (width, n * hidden), 0.02, partition_dim=None, rank=0,
                                                       world=1, device=device or "cpu", dtype=torch.float32))
        base = torch.zeros(width)
        base[2 * n:] = (4.0 * torch.eye(n)).flatten()  # start close to "every stream keeps itself"
        self.base = nn.Parameter(base.to(device or "cpu"))
        self.scale = nn.Parameter(torch.full((3,), float(gate_init), device=device))
        for p in (self.fn, self.base, self.scale):
            PL.mark_tp(p, None, sequence_parallel=sequence_parallel)

    def maps(self, xs: torch.Tensor):
        """xs [T, n, C] -> (pre [T, n], post [T, n], res [T, n, n])."""
        T, n = xs.shape[0], self.n
        flat = xs.reshape(T, -1).float()
        flat = flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + self.eps)
        dyn = flat @ self.fn.t()
        pre = torch.sigmoid(self.scale[0] * dyn[:, :n] + self.base[:n])
        post = 2.0 * torch.sigmoid(self.scale[1] * dyn[:, n:2 * n] + self.base[n:2 * n])
        res = sinkhorn((self.scale[2] * dyn[:, 2 * n:] + self.base[2 * n:]).view(T, n, n), self.iters)
        return pre, post, res

    def read(self, xs: torch.Tensor):
        pre, post, res = self.maps(xs)
        h = torch.einsum("tn,tnc->tc", pre, xs.float()).to(xs.dtype)
        return h, (post, res)

    def write(self, xs: torch.Tensor, out: torch.Tensor, maps) -> torch.Tensor:
        post, res = maps
        mixed = torch.einsum("tmn,tnc->tmc", res, xs.float())
        return (mixed + post.unsqueeze(-1) * out.float().unsqueeze(1)).to(xs.dtype)


class HyperHead(nn.Module):
    """Streams [T, n, C] -> [T, C] with token-dependent sigmoid weights."""

    def __init__(self, hidden: int, n: int, gate_init: float, eps: float, key: str, device=None,
                 sequence_parallel: bool = False):
        super().__init__()
        self.n, self.eps = n, eps
        self.fn = nn.Parameter(PL.init_full_then_slice(key + ".fn", (n, n * hidden), 0.02, partition_dim=None, rank=0,
                                                       world=1, device=device or "cpu", dtype=torch.float32))
        self.base = nn.Parameter(torch.zeros(n, device=device))
        self.scale = nn.Parameter(torch.full((1,), float(gate_init), device=device))
        for p in (self.fn, self.base, self.scale):
            PL.mark_tp(p, None, sequence_parallel=sequence_parallel)

    def forward(self, xs: torch.Tensor) -> torch.Tensor:
        T = xs.shape[0]
        flat = xs.reshape(T, -1).float()
        flat = flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + self.eps)
        w = torch.sigmoid(self.scale * (flat @ self.fn.t()) + self.base)
        return torch.einsum("tn,tnc->tc", w, xs.float()).to(xs.dtype)
