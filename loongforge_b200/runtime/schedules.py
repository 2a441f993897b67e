"""Micro-batch schedules: no pipelining, 1F1B, and interleaved 1F1B (virtual stages).

Plays the role of Megatron's ``get_forward_backward_func`` that the reference calls at
loongforge/train/training_utils.py:2566,1708-1718. Pipeline activations travel as
``[T(/tp under SP), hidden]`` tensors in the pipeline dtype over NCCL/gloo point-to-point
(``batch_isend_irecv``), which stays on the library by design: it is latency- not
bandwidth-bound, and the sends overlap with the next micro-batch's compute.

Contract of ``forward_step_func(data_iterator, model) -> (output, loss_func)``:
``loss_func(output) -> (loss, metrics_dict)``, where ``loss`` is already divided so that the
SUM over micro-batches is the step's loss (the schedule does not rescale).
"""
from __future__ import annotations

import contextlib
import itertools
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from ..parallel import state as ps


def get_forward_backward_func(pp_size: Optional[int] = None, vpp: Optional[int] = None) -> Callable:
    st = ps.get_state()
    pp = st.dims.pp if pp_size is None else pp_size
    vpp = st.dims.vpp if vpp is None else vpp
    if pp <= 1:
        return forward_backward_no_pipelining
    if vpp and vpp > 1:
        return forward_backward_pipelining_interleaved
    return forward_backward_pipelining_1f1b


def _no_sync(model):
    m = model[0] if isinstance(model, (list, tuple)) else model
    return m.no_sync() if hasattr(m, "no_sync") else contextlib.nullcontext()


def _unwrap(model):
    return model.module if hasattr(model, "module") else model


def forward_backward_no_pipelining(*, forward_step_func, data_iterator, model, num_microbatches: int,
                                   forward_only: bool = False, **_) -> List[dict]:
    if isinstance(model, (list, tuple)):
        model = model[0]
    reports = []

    def one(last: bool):
        output, loss_func = forward_step_func(data_iterator, model)
        loss, rep = loss_func(output)
        reports.append(rep)
        if not forward_only:
            loss.backward()

    ctx = _no_sync(model) if not forward_only else contextlib.nullcontext()
    with ctx:
        for _ in range(num_microbatches - 1):
            one(False)
    one(True)
    return reports


# ------------------------------------------------------------------------- p2p helpers
class P2P:
    """Send/recv of activation tensors between adjacent pipeline stages."""

    def __init__(self, shape, dtype, device):
        self.shape, self.dtype, self.device = tuple(shape), dtype, device
        self.st = ps.get_state()
        self.group = self.st.group("pp")

    def _ops(self, send_prev=None, send_next=None, recv_prev=False, recv_next=False):
        st = self.st
        ops, rp, rn = [], None, None
        if recv_prev:
            rp = torch.empty(self.shape, dtype=self.dtype, device=self.device, requires_grad=True)
        if recv_next:
            rn = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        # order ops so that neighbouring ranks post matching send/recv first (avoids deadlock on gloo)
        even = st.pp_rank % 2 == 0
        items = []
        if send_next is not None:
            items.append(("s", send_next.contiguous(), st.pp_next()))
        if recv_prev:
            items.append(("r", rp, st.pp_prev()))
        if send_prev is not None:
            items.append(("s", send_prev.contiguous(), st.pp_prev()))
        if recv_next:
            items.append(("r", rn, st.pp_next()))
        if not even:
            items = [i for i in items if i[0] == "r"] + [i for i in items if i[0] == "s"]
        for kind, t, peer in items:
            ops.append(dist.P2POp(dist.isend if kind == "s" else dist.irecv, t.detach() if kind == "s" else t.data,
                                  peer, self.group))
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        return rp, rn

    def recv_forward(self):
        if self.st.is_first_stage:
            return None
        return self._ops(recv_prev=True)[0]

    def recv_backward(self):
        if self.st.is_last_stage:
            return None
        return self._ops(recv_next=True)[1]

    def send_forward(self, out):
        if not self.st.is_last_stage:
            self._ops(send_next=out)

    def send_backward(self, grad):
        if not self.st.is_first_stage:
            self._ops(send_prev=grad)

    def send_forward_recv_backward(self, out):
        if self.st.is_last_stage:
            return None
        return self._ops(send_next=out, recv_next=True)[1]

    def send_backward_recv_forward(self, grad):
        if self.st.is_first_stage:
            return None
        return self._ops(send_prev=grad, recv_prev=True)[0]


def _forward_one(forward_step_func, data_iterator, model, input_tensor, reports, is_last_stage):
    _unwrap(model).set_input_tensor(input_tensor)
    output, loss_func = forward_step_func(data_iterator, model)
    if is_last_stage:
        loss, rep = loss_func(output)
        reports.append(rep)
        return loss
    return output


def _backward_one(input_tensor, output_tensor, output_grad):
    if input_tensor is not None:
        input_tensor.retain_grad()
    if output_grad is None:
        output_tensor.backward()
    else:
        torch.autograd.backward(output_tensor, grad_tensors=output_grad)
    return input_tensor.grad if input_tensor is not None else None


def forward_backward_pipelining_1f1b(*, forward_step_func, data_iterator, model, num_microbatches: int,
                                     tensor_shape, dtype, forward_only: bool = False, **_) -> List[dict]:
    """Non-interleaved 1F1B: warm-up forwards, steady 1F1B, cool-down backwards."""
    if isinstance(model, (list, tuple)):
        model = model[0]
    st = ps.get_state()
    device = next(model.parameters()).device
    p2p = P2P(tensor_shape, dtype, device)
    warm = min(st.dims.pp - st.pp_rank - 1, num_microbatches)
    remaining = num_microbatches - warm
    inputs, outputs, reports = [], [], []
    sync_ctx = _no_sync(model) if not forward_only else contextlib.nullcontext()
    sync_ctx.__enter__()
    entered = True

    def enable_sync():
        nonlocal entered
        if entered:
            sync_ctx.__exit__(None, None, None)
            entered = False

    for _ in range(warm):
        inp = p2p.recv_forward()
        out = _forward_one(forward_step_func, data_iterator, model, inp, reports, st.is_last_stage)
        p2p.send_forward(out)
        if not forward_only:
            inputs.append(inp)
            outputs.append(out)
    inp = p2p.recv_forward() if remaining > 0 else None
    for i in range(remaining):
        last_iter = i == remaining - 1
        out = _forward_one(forward_step_func, data_iterator, model, inp, reports, st.is_last_stage)
        if forward_only:
            p2p.send_forward(out)
            if not last_iter:
                inp = p2p.recv_forward()
            continue
        out_grad = p2p.send_forward_recv_backward(out)
        inputs.append(inp)
        outputs.append(out)
        bi, bo = inputs.pop(0), outputs.pop(0)
        if warm == 0 and last_iter:
            enable_sync()
        in_grad = _backward_one(bi, bo, out_grad)
        if last_iter:
            inp = None
            p2p.send_backward(in_grad)
        else:
            inp = p2p.send_backward_recv_forward(in_grad)
    if not forward_only:
        for i in range(warm):
            if i == warm - 1:
                enable_sync()
            bi, bo = inputs.pop(0), outputs.pop(0)
            out_grad = p2p.recv_backward()
            in_grad = _backward_one(bi, bo, out_grad)
            p2p.send_backward(in_grad)
    enable_sync()
    return reports


def forward_backward_pipelining_interleaved(*, forward_step_func, data_iterator, model, num_microbatches: int,
                                            tensor_shape, dtype, forward_only: bool = False, **_) -> List[dict]:
    """Interleaved 1F1B over virtual pipeline stages: each rank holds `v` model chunks; the `pp * v` virtual stages
    form a ring (chunk c on the last rank feeds chunk c+1 on the first rank).

    Work is cut into units (chunk, micro-batch). Micro-batches go in groups of `pp`; the FORWARD stream visits, per
    group, chunk 0 for its pp micro-batches, then chunk 1, ...; the BACKWARD stream visits the same units with the
    chunks in reverse. Both streams advance in lock step: at tick t rank r runs forward unit ``t - r`` and backward
    unit ``t - v*pp - (pp-1-r)`` (whichever exist), then posts ALL its sends and receives for the next tick - forward
    activation to the next rank, gradient to the previous rank, and the matching receives - as one batch of
    non-blocking operations. No rank ever blocks in a send whose receiver is blocked in a send, which a rendezvous
    transport (gloo, NCCL point-to-point) needs with wrap-around neighbours. The backward stream starts `v*pp` ticks
    after the forward stream (when the last rank has finished the first group's last chunk), so a rank holds at most
    ``v*pp + pp - 1 - 2r`` units' activations, and the pipeline fills and drains once per step, not once per group."""
    assert isinstance(model, (list, tuple)) and len(model) > 1
    st = ps.get_state()
    pp, v, r = st.dims.pp, len(model), st.pp_rank
    device = next(model[0].parameters()).device
    p2p = P2P(tensor_shape, dtype, device)
    # every chunk must see the SAME sequence of micro-batches (the first chunk embeds the tokens whose labels the
    # last chunk scores); a single iterator is therefore split into v buffered views, each drained by one chunk
    iters = list(data_iterator) if isinstance(data_iterator, (list, tuple)) else list(itertools.tee(data_iterator, v))
    reports: List[dict] = []
    assert num_microbatches % pp == 0, "interleaved schedule needs num_microbatches divisible by pp"
    total, group = num_microbatches * v, v * pp
    t0 = group  # delay of the backward stream
    ticks = total + pp - 1 if forward_only else total + t0 + pp - 1

    def set_last(m, flag):
        if hasattr(m, "is_last_microbatch"):
            m.is_last_microbatch = flag

    def unit(u, backward):
        """(chunk, micro-batch, first virtual stage?, last virtual stage?) of stream position u, or None."""
        if not 0 <= u < total:
            return None
        g, rem = divmod(u, group)
        c, m = divmod(rem, pp)
        if backward:
            c = v - 1 - c
        return c, g * pp + m, st.is_first_stage and c == 0, st.is_last_stage and c == v - 1

    f_unit = lambda t: unit(t - r, False)  # noqa: E731
    b_unit = lambda t: None if forward_only else unit(t - t0 - (pp - 1 - r), True)  # noqa: E731
    saved = {}
    inp, out_grad = None, None
    for m in model:
        set_last(m, False)
    for t in range(ticks):
        out = in_grad = None
        cur = f_unit(t)
        if cur is not None:
            c, mb, first_virtual, last_virtual = cur
            x = None if first_virtual else inp
            out = _forward_one(forward_step_func, iters[c], model[c], x, reports, last_virtual)
            if not forward_only:
                saved[(c, mb)] = (x, out)
            if last_virtual:
                out = None
        cur = b_unit(t)
        if cur is not None:
            c, mb, first_virtual, last_virtual = cur
            b_in, b_out = saved.pop((c, mb))
            # gradient buckets of chunk c may start reducing only on its very last backward
            set_last(model[c], mb == num_microbatches - 1)
            in_grad = _backward_one(b_in, b_out, None if last_virtual else out_grad)
            if first_virtual:
                in_grad = None
        nf, nb = f_unit(t + 1), b_unit(t + 1)
        inp, out_grad = p2p._ops(send_next=out, recv_prev=nf is not None and not nf[2],
                                 send_prev=in_grad, recv_next=nb is not None and not nb[3])
    assert not saved, "every forward unit must have had its backward"
    for m in model:
        set_last(m, True)
    return reports
