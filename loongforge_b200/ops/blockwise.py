"""Row-blocked evaluation with recomputation in backward.

Gather-based sparse attention (DSA top-k attention, compressed sparse attention) materialises ``[rows, K, d]`` gathered
keys per query block. Under plain autograd every block's intermediates stay alive until backward — tens of GB per layer
at 8k tokens. ``blockwise_apply`` runs ``fn`` on row blocks WITHOUT recording the graph and, in backward, recomputes one
block at a time with autograd and back-propagates that block's output gradient, so peak memory is that of one block.
This is what lets the PyTorch formulation of the sparse paths train at long sequence lengths (the reference reaches the
same end with hand-written fused kernels that never materialise the gathered tensor)."""
from __future__ import annotations

from typing import Callable, Sequence, Tuple

import torch


class _BlockwiseFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, block, n_rowwise, *tensors):
        rowwise, shared = tensors[:n_rowwise], tensors[n_rowwise:]
        rows = rowwise[0].shape[0]
        outs = []
        with torch.no_grad():
            for s in range(0, rows, block):
                outs.append(fn(*[t[s:s + block] for t in rowwise], *shared))
        ctx.fn, ctx.block, ctx.n_rowwise = fn, block, n_rowwise
        ctx.save_for_backward(*tensors)
        return torch.cat(outs, 0)

    @staticmethod
    def backward(ctx, grad_out):
        tensors = ctx.saved_tensors
        n = ctx.n_rowwise
        rowwise, shared = tensors[:n], tensors[n:]
        rows = rowwise[0].shape[0]
        need = ctx.needs_input_grad[3:]
        shared_leaves = [t.detach().requires_grad_(bool(need[n + i]) and t.is_floating_point()) for i, t in enumerate(shared)]
        row_grads = [torch.zeros_like(t) if (need[i] and t.is_floating_point()) else None for i, t in enumerate(rowwise)]
        for s in range(0, rows, ctx.block):
            e = min(rows, s + ctx.block)
            blk = [t[s:e].detach().requires_grad_(row_grads[i] is not None) for i, t in enumerate(rowwise)]
            with torch.enable_grad():
                out = ctx.fn(*blk, *shared_leaves)
            if out.requires_grad:
                torch.autograd.backward(out, grad_out[s:e])  # accumulates into shared_leaves[i].grad
            for i, b in enumerate(blk):
                if row_grads[i] is not None and b.grad is not None:
                    row_grads[i][s:e] = b.grad
        shared_grads = [(t.grad if t.requires_grad else None) for t in shared_leaves]
        return (None, None, None, *row_grads, *shared_grads)


def blockwise_apply(fn: Callable[..., torch.Tensor], rowwise: Sequence[torch.Tensor], shared: Sequence[torch.Tensor],
                    block: int) -> torch.Tensor:
    """``cat([fn(*[t[s:s+block] for t in rowwise], *shared) for s in ...])`` with O(block) activation memory.
    `fn` must be a pure function of its tensor arguments and return one tensor with the block's rows first."""
    return _BlockwiseFn.apply(fn, int(block), len(rowwise), *rowwise, *shared)
