"""ChunkPipe: a long sequence is cut into chunks that run through the layers one after another, each chunk attending to
the cached keys / values of the chunks before it; activations of only ONE chunk are alive at a time.

Forward pass (no autograd): chunk c computes its K/V per layer, appends them to the caches, produces its loss.
Backward pass, chunks in REVERSE order: chunk c is recomputed with autograd against the caches of chunks < c (leaf
tensors), its loss is back-propagated together with the gradient that later chunks deposited on ITS keys / values,
and the gradient it produces for earlier chunks' K/V is accumulated into their cache gradients — the cross-chunk
gradient accumulation of the reference (loongforge/train/training_utils.py:1696-1706 micro-batch x chunk counting,
chunk-aware RoPE offsets and recompute in base_gpt_model.py / language_transformer_block.py).

``ChunkedAttentionLayer`` is the protocol a layer must follow (``forward(x, past_kv, offset) -> (y, (k, v))``);
``CausalSelfAttentionBlock`` is a reference layer used by the tests and by small models."""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

KV = Tuple[torch.Tensor, torch.Tensor]


class CausalSelfAttentionBlock(nn.Module):
    """Pre-norm attention + MLP block over ``[T, C]`` tokens with an optional key/value prefix."""

    def __init__(self, dim: int, heads: int, rope_theta: float = 10000.0):
        super().__init__()
        self.h, self.d = heads, dim // heads
        self.n1, self.n2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.qkv, self.o = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.mlp = nn.Sequential(nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))
        self.theta = rope_theta

    def _rope(self, x, offset):
        T = x.shape[0]
        inv = 1.0 / (self.theta ** (torch.arange(0, self.d, 2, dtype=torch.float32) / self.d))
        ang = torch.outer(torch.arange(offset, offset + T, dtype=torch.float32), inv)
        cos, sin = ang.cos()[:, None], ang.sin()[:, None]
        a, b = x[..., :self.d // 2], x[..., self.d // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    def forward(self, x: torch.Tensor, past: Optional[KV] = None, offset: int = 0):
        T = x.shape[0]
        q, k, v = self.qkv(self.n1(x)).view(T, 3, self.h, self.d).unbind(1)
        q, k = self._rope(q, offset), self._rope(k, offset)
        if past is not None:
            kk, vv = torch.cat([past[0], k], 0), torch.cat([past[1], v], 0)
        else:
            kk, vv = k, v
        P = kk.shape[0] - T
        mask = torch.ones(T, P + T, dtype=torch.bool).tril(P)  # token i sees the whole prefix and itself
        o = F.scaled_dot_product_attention(q.transpose(0, 1), kk.transpose(0, 1), vv.transpose(0, 1), attn_mask=mask)
        x = x + self.o(o.transpose(0, 1).reshape(T, -1))
        return x + self.mlp(self.n2(x)), (k, v)


def chunk_bounds(seq_len: int, num_chunks: int) -> List[Tuple[int, int]]:
    size = math.ceil(seq_len / num_chunks)
    return [(s, min(s + size, seq_len)) for s in range(0, seq_len, size)]


def chunkpipe_forward_backward(layers: Sequence[nn.Module], embed: Optional[Callable[[torch.Tensor], torch.Tensor]],
                               loss_fn: Optional[Callable[[torch.Tensor, int, int], torch.Tensor]], tokens: torch.Tensor,
                               num_chunks: int, p2p=None) -> float:
    """Accumulates parameter gradients of ``sum_c loss_fn(hidden_c, start_c, end_c)`` and returns the loss value.
    Peak activation memory is that of one chunk plus the K/V caches.

    With pipeline parallelism (`p2p`: the stage-to-stage send / receive helper of ``runtime/schedules.py``) `layers`
    are THIS stage's layers and the chunks flow through the stages like micro-batches: in the forward phase stage s
    works on chunk c while stage s + 1 works on chunk c - 1, in the backward phase the same in reverse chunk order.
    Every stage keeps the K/V caches of its own layers and the chunk inputs it received (one sequence of activations
    in total); `embed` is used on the first stage only, `loss_fn` on the last (other stages return 0)."""
    first = p2p is None or p2p.st.is_first_stage
    last = p2p is None or p2p.st.is_last_stage
    bounds = chunk_bounds(tokens.shape[0], num_chunks)
    if p2p is not None and len({e - s for s, e in bounds}) != 1:
        raise ValueError("with pipeline parallelism all chunks must have the same length")
    L = len(layers)
    caches: List[List[KV]] = [[] for _ in range(L)]  # caches[l][c] = (k, v) of chunk c at layer l
    received: List[Optional[torch.Tensor]] = []      # chunk inputs of a later stage, kept for the recomputation
    total = 0.0
    with torch.no_grad():
        for (s, e) in bounds:
            if first:
                x = embed(tokens[s:e])
            else:
                x = p2p.recv_forward().detach()
                received.append(x)
            for l, layer in enumerate(layers):
                past = (torch.cat([kv[0] for kv in caches[l]]), torch.cat([kv[1] for kv in caches[l]])) if caches[l] else None
                x, kv = layer(x, past, s)
                caches[l].append(kv)
            if last:
                total += float(loss_fn(x, s, e))
            else:
                p2p.send_forward(x)
    grads: List[List[Optional[KV]]] = [[None] * len(bounds) for _ in range(L)]  # gradient deposited on chunk c's K/V
    for c in range(len(bounds) - 1, -1, -1):
        s, e = bounds[c]
        leaves: List[Optional[KV]] = []
        if first:
            x_in = None
            x = embed(tokens[s:e])
        else:
            x_in = received[c].detach().requires_grad_(True)
            x = x_in
        own: List[KV] = []
        for l, layer in enumerate(layers):
            if c > 0:
                pk = torch.cat([caches[l][j][0] for j in range(c)]).requires_grad_(True)
                pv = torch.cat([caches[l][j][1] for j in range(c)]).requires_grad_(True)
                leaves.append((pk, pv))
                x, kv = layer(x, (pk, pv), s)
            else:
                leaves.append(None)
                x, kv = layer(x, None, s)
            own.append(kv)
        if last:
            outs, outg = [loss_fn(x, s, e)], [None]
        else:
            outs, outg = [x], [p2p.recv_backward()]
        for l in range(L):
            if grads[l][c] is not None:  # what later chunks want from this chunk's keys / values
                outs += [own[l][0], own[l][1]]
                outg += [grads[l][c][0], grads[l][c][1]]
        torch.autograd.backward(outs, outg)
        if not first:
            p2p.send_backward(x_in.grad)
            received[c] = None
        for l in range(L):
            if leaves[l] is None:
                continue
            gk, gv = leaves[l][0].grad, leaves[l][1].grad
            off = 0
            for j in range(c):
                n = caches[l][j][0].shape[0]
                piece = (gk[off:off + n], gv[off:off + n])
                grads[l][j] = piece if grads[l][j] is None else (grads[l][j][0] + piece[0], grads[l][j][1] + piece[1])
                off += n
        for l in range(L):
            caches[l][c] = (caches[l][c][0], caches[l][c][1])  # keep for earlier chunks' recomputation
            grads[l][c] = None
    return total


def num_microbatches_with_chunks(num_microbatches: int, num_chunks: int) -> int:
    """The pipeline schedule sees every chunk as a micro-batch of its own."""
    return num_microbatches * num_chunks


# ----------------------------------------------------------------------------- GPT models
def gpt_chunkpipe_step(model: nn.Module, tokens: torch.Tensor, position_ids: torch.Tensor, labels: torch.Tensor,
                       loss_mask: torch.Tensor, num_chunks: int, loss_scale: float) -> torch.Tensor:
    """One micro-batch (ONE sequence, flat ``[T]`` tensors) of a GPT model (one pipeline stage of it, when the model is
    pipeline parallel: chunks then flow through the stages like micro-batches) through the chunk pipeline:
    accumulates the gradients of ``loss_scale * sum(loss * mask)`` and returns that loss value. Attention layers
    take the earlier chunks' keys / values through ``models.transformer.CHUNK_PREFIX`` (multi-latent attention: the
    materialised per-head keys / values in its dense form, the 576-value compressed keys and the indexer keys in its
    sparse form, as the reference caches them: dsa_fused.py:240-421); every other sub-layer (norms,
    dense and MoE MLPs, the fused linear + cross-entropy head) is token-local and runs on the chunk alone. Tensor
    parallelism (with or without sequence parallelism) needs nothing extra: every rank caches the keys / values of its
    own heads."""
    from ..models import transformer as TF

    cfg = model.cfg
    assert not (cfg.enable_hyper_connections or cfg.csa_compress_ratios or cfg.layer_types
                or cfg.full_attention_interval or cfg.mtp_num_layers), \
        "chunk pipelining covers softmax-attention and multi-latent (dense or sparse) attention GPT layers"
    assert not (cfg.use_dsa and (cfg.dsa_indexer_topk_freq or 1) > 1), \
        "chunk pipelining does not carry shared top-k indices (IndexShare) from layer to layer"
    dev = tokens.device
    mask_f = loss_mask.float()
    from ..parallel import state as ps
    st = ps.get_state(model.state_name)
    sp_factor = st.dims.tp if (cfg.sequence_parallel and st.dims.tp > 1) else 1
    bounds = chunk_bounds(tokens.shape[0], num_chunks)
    if any((e - s) % sp_factor for s, e in bounds):
        raise ValueError("with sequence parallelism every chunk length must divide by the tensor-parallel size")

    class _Layer:
        def __init__(self, layer):
            self.layer = layer

        def __call__(self, x, past, offset):
            T = x.shape[0] * sp_factor  # under sequence parallelism x is this rank's shard of the chunk
            rotary = model.build_rotary(position_ids[..., offset:offset + T], position_ids.shape[-1], dev)
            TF.CHUNK_PREFIX.update(active=True, past=past, out=None)
            try:
                y = self.layer(x, rotary, None)
                return y, TF.CHUNK_PREFIX["out"]
            finally:
                TF.CHUNK_PREFIX.update(active=False, past=None, out=None)

    def loss_fn(hidden, s, e):
        if model.decoder.final_layernorm is not None:
            hidden = model.decoder.final_layernorm(hidden)
        losses = model.postprocess(hidden, labels[s:e], loss_mask[s:e], loss_scale)
        return (losses * mask_f[s:e]).sum() * loss_scale

    p2p = None
    if st.dims.pp > 1:
        from .schedules import P2P
        width = cfg.hidden_size * (cfg.num_residual_streams if cfg.enable_hyper_connections else 1)
        p2p = P2P(((bounds[0][1] - bounds[0][0]) // sp_factor, width), cfg.params_dtype, dev)
    total = chunkpipe_forward_backward([_Layer(l) for l in model.decoder.layers],
                                       model.embed if model.pre_process else None,
                                       loss_fn if model.post_process else None, tokens, num_chunks, p2p=p2p)
    return torch.tensor(total, device=dev)
