"""Training runtime: model/optimizer set-up, the train step, the logging line and the loop.

Counterpart of the reference's ``pretrain()`` / ``setup_model_and_optimizer()`` / ``train_step()``
/ ``training_log()`` (loongforge/train/training_utils.py:345,1030,1471,2001,2431). The public
entry points are ``Trainer`` (programmatic) and ``loongforge_b200.train`` (CLI).
"""
from __future__ import annotations

import copy
import dataclasses
import math
import os
import time
from typing import Callable, Dict, Iterator, List, Optional

import torch
import torch.distributed as dist

from ..models.config import TransformerConfig
from ..models.gpt import GPTModel, pipeline_layer_split
from ..models.transformer import PackedSeqParams
from ..optim.lr_scheduler import OptimizerParamScheduler
from ..parallel import state as ps
from ..parallel.ddp import DDPConfig, DistributedDataParallel
from ..parallel.dist_optimizer import DistributedOptimizer, OptimizerConfig
from ..parallel.state import ParallelDims
from . import schedules
from .microbatches import MicrobatchCalculator
from .timers import Timers


@dataclasses.dataclass
class TrainConfig:
    micro_batch_size: int = 1
    global_batch_size: int = 8
    seq_length: int = 128
    train_iters: int = 20
    lr: float = 1e-4
    min_lr: float = 0.0
    lr_decay_style: str = "constant"
    lr_warmup_iters: int = 0
    rampup_batch_size: Optional[List[int]] = None  # (start, increment, ramp samples): global batch size grows to its final value
    lr_decay_iters: Optional[int] = None
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    bf16: bool = False
    seed: int = 1234
    log_interval: int = 1
    save: Optional[str] = None
    load: Optional[str] = None
    save_interval: Optional[int] = None
    ckpt_format: str = "torch_dist"
    use_distributed_optimizer: bool = True
    overlap_grad_reduce: bool = True
    overlap_param_gather: bool = False
    grad_reduce_in_fp32: bool = True
    exp_avg_dtype: torch.dtype = torch.float32
    exp_avg_sq_dtype: torch.dtype = torch.float32
    master_as_remainder: bool = False
    timing_log_level: int = 0  # 0 | 1 | 2, see Trainer.timers
    log_timers_to_tensorboard: bool = False  # phase times also go to the scalar writers
    optimizer_cpu_offload: bool = False  # masters + Adam moments on the host, native host AdamW
    optimizer_offload_fraction: float = 1.0  # part of the optimizer state (whole shards) that goes to the host
    optimizer: str = "adam"  # adam | sgd
    sgd_momentum: float = 0.9
    fp8_policy_file: Optional[str] = None  # JSON rules: which linear kinds run FP8 (runtime/fp8_policy.py)
    log_memory_stats: bool = False  # memory fields in the log line also on the host (they are always there on GPUs)
    no_save_optim: bool = False  # checkpoints without optimizer state / RNG state
    no_save_rng: bool = False
    eval_interval: int = 0  # > 0: run `eval_iters` forward-only steps on the validation stream every N iterations
    eval_iters: int = 0
    rerun_mode: str = "disabled"  # disabled | validate_results | report_stats (runtime/resilience.py)
    error_injection_rate: int = 0  # host-side loss corruption every N steps on average (testing the rerun machine)
    error_injection_type: str = "transient_error"
    iterations_to_skip: Optional[List[int]] = None  # their data is consumed, no update happens
    check_weight_hash_interval: int = 0  # > 0: compare parameter checksums across data-parallel replicas every N steps
    dp_balance: bool = False  # trade whole micro-batches between DP ranks by modelled cost (data/dp_balance.py)
    chunkpipe_chunks: int = 0  # > 1: every sequence runs as that many chunks (runtime/chunkpipe.py)
    overlap_moe_expert_parallel_comm: bool = False  # 1F1B interleave of MoE exchanges and compute (runtime/a2a_overlap.py)
    use_fsdp: bool = False  # FSDP2 units instead of DDP + distributed optimizer (runtime/fsdp_trainer.py)
    fsdp_sharding_strategy: str = "optim_grads_params"  # or optim_grads
    ddp_bucket_size: Optional[int] = None
    calculate_per_token_loss: bool = False
    custom_pipeline_layers: Optional[List[int]] = None
    custom_pipeline_recompute_layers: Optional[List[int]] = None  # recomputed layers per pipeline stage
    training_phase: str = "pretrain"
    log_throughput: bool = True
    check_for_nan_in_loss: bool = True
    exit_on_nan: bool = False
    async_save: bool = False
    peer_optimizer: bool = False  # grad reduce-scatter / param all-gather inside the optimizer kernels (peer memory)
    freeze_parameters: Optional[List[str]] = None  # parameter-name prefixes that do not train (--freeze-parameters)
    freeze_parameters_regex: Optional[str] = None  # ... or a regular expression over the full parameter name
    trainable_modules: Optional[List[str]] = None  # if given (and not ["all"]): only names containing one of these train


def _device_for_rank() -> torch.device:
    if torch.cuda.is_available():
        local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local)
        return torch.device("cuda", local)
    return torch.device("cpu")


def init_distributed(backend: Optional[str] = None, timeout_s: int = 1800) -> torch.device:
    """torchrun-style rendezvous (RANK / WORLD_SIZE / MASTER_*); also accepts OpenMPI variables
    as the reference does (loongforge/train/parser.py:101-106)."""
    dev = _device_for_rank()
    if "RANK" not in os.environ and "OMPI_COMM_WORLD_RANK" in os.environ:
        os.environ["RANK"] = os.environ["OMPI_COMM_WORLD_RANK"]
        os.environ["WORLD_SIZE"] = os.environ["OMPI_COMM_WORLD_SIZE"]
        os.environ.setdefault("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        import datetime
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        be = backend or ("nccl" if dev.type == "cuda" else "gloo")
        kw = {}
        if be == "nccl":
            kw["device_id"] = dev
        dist.init_process_group(be, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return dev


class Trainer:
    """Owns model chunks, DDP wrappers, optimizer, scheduler and the step function."""

    def __init__(self, model_cfg: TransformerConfig, train_cfg: TrainConfig, dims: Optional[ParallelDims] = None,
                 *, device: Optional[torch.device] = None, model_provider: Optional[Callable] = None,
                 forward_step: Optional[Callable] = None):
        self.mcfg, self.tcfg = model_cfg, train_cfg
        self.device = device or _device_for_rank()
        dims = dims or ParallelDims()
        if not ps.model_parallel_is_initialized():
            ps.initialize_model_parallel(dims, gloo_groups=False)
            from ..parallel.context_parallel import ensure_cp_groups
            ensure_cp_groups()
        self.st = ps.get_state()
        self.world = self.st.world_size
        self.dp = self.st.dp_size
        # level 0: only the iteration time of the log line; 1: forward-backward and optimizer, timed with a device
        # synchronisation on both sides; 2: also the smaller phases
        self.timers = Timers(log_level=train_cfg.timing_log_level, device_sync=True)
        if train_cfg.bf16:
            model_cfg.params_dtype = torch.bfloat16
        # default stream alike on the TP ranks of a stage (dropout on replicated activations), tracked streams that
        # differ per TP / expert rank (dropout on sharded activations)
        from ..parallel.random import model_parallel_manual_seed
        model_parallel_manual_seed(train_cfg.seed, self.st.tp_rank, self.st.pp_rank, self.st.ep_rank)
        from ..parallel.layers import set_init_seed
        set_init_seed(train_cfg.seed)
        self.mb_calc = MicrobatchCalculator(train_cfg.global_batch_size, train_cfg.micro_batch_size, self.dp,
                                            rampup=train_cfg.rampup_batch_size)
        self.model_provider = model_provider or self._default_model_provider
        self.forward_step = forward_step or self._default_forward_step
        self.models = self._build_models()
        from .resilience import ErrorInjector, RerunStateMachine
        self.rerun = RerunStateMachine(train_cfg.rerun_mode)
        self.injector = (ErrorInjector(train_cfg.error_injection_rate, train_cfg.error_injection_type, train_cfg.seed)
                         if train_cfg.error_injection_rate > 0 else None)
        self.exit_requested: Optional[str] = None
        self.fp8_decisions = {}
        if model_cfg.fp8:
            from . import fp8_policy as FP
            policy = FP.FP8Policy.from_json(train_cfg.fp8_policy_file) if train_cfg.fp8_policy_file else FP.default_policy()
            tokens = train_cfg.seq_length * train_cfg.micro_batch_size // max(self.st.dims.cp, 1)
            for m in self.models:
                self.fp8_decisions.update(FP.apply_fp8_policy(m.module, policy, tokens, self.st.dims.tp))
        self.optimizer = self._build_optimizer()
        self._shared_embeddings = [p for m in self.models for p in m.module.parameters()
                                   if getattr(p, "shared_embedding", False)]
        if self._shared_embeddings and self.st.group("embd") is not None:
            # start from identical copies on the first and last pipeline stage, then keep them identical by summing
            # their gradients after every data-parallel reduction
            with torch.no_grad():
                for p in self._shared_embeddings:
                    dist.broadcast(p.data, src=self.st.group_ranks["embd"][0], group=self.st.group("embd"))
            self.optimizer.reload_model_params()
            self.optimizer.post_sync_hooks.append(self._allreduce_embedding_grads)
        # Gradients that are partial sums over the tensor-parallel group are completed AFTER the data-parallel
        # reduction has finished: with an overlapped reduction the last buckets are still being reduced in place on
        # the communication stream when backward returns, and touching them earlier would race with it.
        self.optimizer.post_sync_hooks.insert(0, self._allreduce_sequence_parallel_grads)
        self.scheduler = OptimizerParamScheduler(
            self.optimizer, max_lr=train_cfg.lr, min_lr=train_cfg.min_lr, warmup_steps=train_cfg.lr_warmup_iters,
            decay_steps=train_cfg.lr_decay_iters or train_cfg.train_iters, decay_style=train_cfg.lr_decay_style)
        self.iteration = 0
        self.consumed_samples = 0
        self.num_flops_so_far = 0.0
        self._skipped = 0
        self._nan = 0

    # ------------------------------------------------------------------ construction
    def _default_model_provider(self, pre_process, post_process, layer_numbers):
        return GPTModel(self.mcfg, pre_process=pre_process, post_process=post_process, layer_numbers=layer_numbers,
                        device=self.device)

    def _build_models(self) -> List[DistributedDataParallel]:
        st = self.st
        pp, vpp = st.dims.pp, st.dims.vpp or 1
        custom = self.tcfg.custom_pipeline_layers
        if custom and len(custom) == pp and vpp > 1:  # counts per pipeline rank -> per virtual stage
            from ..parallel.pipeline_layout import split_rank_layers_over_virtual_stages
            custom = split_rank_layers_over_virtual_stages(custom, vpp)
        splits = pipeline_layer_split(self.mcfg.num_layers, pp * vpp, custom)
        rec = self.tcfg.custom_pipeline_recompute_layers
        if rec:
            # per-stage number of recomputed layers (stages near the pipeline's start hold more activations in flight)
            self.mcfg = copy.copy(self.mcfg)
            self.mcfg.recompute_granularity = "full"
            self.mcfg.recompute_method = self.mcfg.recompute_method or "block"
            self.mcfg.recompute_num_layers = rec[st.pp_rank]
        chunks = []
        for v in range(vpp):
            virt = v * pp + st.pp_rank
            module = self.model_provider(virt == 0, virt == pp * vpp - 1, splits[virt])
            self._apply_freezing(module)
            # The NCCL all-to-all dispatcher puts expert-parallel collectives on the compute stream during backward;
            # an overlapped gradient reduce-scatter would run a SECOND communicator (the data-parallel one) next to
            # them on another stream, in an order that differs between ranks. That combination stopped making progress
            # at 8 expert-parallel ranks, so with that dispatcher the reduction waits for the end of backward. The
            # peer-memory dispatcher issues no NCCL call in backward and keeps the overlap.
            serial_nccl = (bool(self.mcfg.num_moe_experts) and st.dims.ep > 1 and self.device.type == "cuda"
                           and self.mcfg.moe_token_dispatcher_type != "peer")
            ddp_cfg = DDPConfig(grad_reduce_in_fp32=self.tcfg.grad_reduce_in_fp32,
                                overlap_grad_reduce=self.tcfg.overlap_grad_reduce and not serial_nccl,
                                use_distributed_optimizer=self.tcfg.use_distributed_optimizer,
                                peer_optimizer=self.tcfg.peer_optimizer,
                                bucket_size=self.tcfg.ddp_bucket_size or max(40_000_000, 1_000_000 * self.dp))
            # bucketing only helps the chunk whose backward runs last (reference: training_utils.py:987-988)
            chunks.append(DistributedDataParallel(module, ddp_cfg, disable_bucketing=v > 0))
        for c in chunks:
            c.broadcast_params()
        return chunks

    def _apply_freezing(self, module) -> int:
        """``--freeze-parameters`` (name prefixes), ``--freeze-parameters-regex`` and ``--trainable-modules``: the
        selected parameters get ``requires_grad = False`` before gradient buffers and optimizer shards are laid out, so
        they cost neither gradient memory nor optimizer state (reference: loongforge/train/arguments.py:309-330)."""
        import re

        t = self.tcfg
        prefixes = [p for p in (t.freeze_parameters or []) if p]
        rx = re.compile(t.freeze_parameters_regex) if t.freeze_parameters_regex else None
        only = [m for m in (t.trainable_modules or []) if m and m != "all"]
        n = 0
        for name, p in module.named_parameters():
            frozen = any(name.startswith(pre) for pre in prefixes) or bool(rx and rx.search(name))
            if only and not any(m in name for m in only):
                frozen = True
            if frozen and p.requires_grad:
                p.requires_grad_(False)
                n += 1
        return n

    def _build_optimizer(self) -> DistributedOptimizer:
        t = self.tcfg
        ocfg = OptimizerConfig(lr=t.lr, min_lr=t.min_lr, weight_decay=t.weight_decay, adam_beta1=t.adam_beta1,
                               adam_beta2=t.adam_beta2, adam_eps=t.adam_eps, clip_grad=t.clip_grad,
                               exp_avg_dtype=t.exp_avg_dtype, exp_avg_sq_dtype=t.exp_avg_sq_dtype,
                               overlap_param_gather=t.overlap_param_gather,
                               master_as_remainder=t.master_as_remainder and t.optimizer != "sgd",
                               cpu_offload=t.optimizer_cpu_offload, offload_fraction=t.optimizer_offload_fraction,
                               optimizer=t.optimizer, sgd_momentum=t.sgd_momentum)
        return DistributedOptimizer(self.models, ocfg)

    # ------------------------------------------------------------------ default LLM pretrain step
    def get_batch(self, data_iterator) -> Dict[str, torch.Tensor]:
        """Pull one micro-batch, move it to the device (H2D from pinned memory) and flatten to the
        packed-token layout. On pipeline-middle stages only position ids are needed."""
        batch = next(data_iterator)
        out = {}
        for k, v in batch.items():
            out[k] = v.to(self.device, non_blocking=True) if isinstance(v, torch.Tensor) else v
        return out

    def _microbatch_inputs(self, b: Dict[str, torch.Tensor]):
        """Batch dict -> (keyword arguments of ``GPTModel.forward``, loss function of the per-token losses)."""
        cp = self.st.dims.cp
        extra = {}
        if cp > 1:
            from ..parallel.context_parallel import get_batch_on_this_cp_rank
            if self.mcfg.mtp_num_layers > 0 and self.st.is_last_stage:
                # multi-token prediction shifts tokens across the chunk boundaries of the context-parallel slice
                extra["full_batch"] = {k: b[k] for k in ("tokens", "labels", "loss_mask")}
            b = get_batch_on_this_cp_rank(b, cp, self.st.cp_rank)
        tokens = b["tokens"].reshape(-1)
        labels = b["labels"].reshape(-1)
        mask = b["loss_mask"].reshape(-1)
        pos = b["position_ids"].reshape(-1)
        bs = b["tokens"].shape[0]
        packed = None
        if bs > 1 or "cu_seqlens" in b:
            cu = b.get("cu_seqlens")
            full_len = b["tokens"].shape[1] * cp  # row length before the context-parallel slice
            if cu is None:
                # one sequence per row; under context parallelism boundaries are offsets in the FULL rows
                cu = torch.arange(0, (bs + 1) * full_len, full_len, dtype=torch.int32, device=self.device)
            packed = PackedSeqParams(cu_seqlens=cu, max_seqlen=full_len,
                                     row_length=full_len if (cp > 1 and bs > 1) else None)
        n_valid = b.get("num_valid_tokens")
        if n_valid is None:
            n_valid = int(mask.numel()) * cp
        nmb = self.mb_calc.num_microbatches
        # each context-parallel rank sums its own tokens; gradients are averaged over dp x cp, so the
        # factor cp turns that average into (sum over cp, mean over dp)
        scale = float(cp) / (max(n_valid, 1) * nmb)

        def loss_func(losses):
            loss = (losses * mask.float()).sum() * scale
            return loss, {"lm loss": loss.detach() * nmb, "num_tokens": n_valid}

        kw = dict(tokens=tokens, position_ids=pos, labels=labels, loss_mask=mask, packed=packed, loss_scale=scale,
                  **extra)
        return kw, loss_func

    def _default_forward_step(self, data_iterator, model):
        kw, loss_func = self._microbatch_inputs(self.get_batch(data_iterator))
        tokens, pos = kw.pop("tokens"), kw.pop("position_ids")
        return model(tokens, pos, **kw), loss_func

    def _a2a_overlap_microbatches(self, data_iterator) -> List[dict]:
        """The step's micro-batches under the MoE all-to-all overlap schedule (``runtime/a2a_overlap.py``): forward of
        micro-batch i is issued node by node between the backward nodes of micro-batch i - 1, expert-parallel
        exchanges on a side stream."""
        from .a2a_overlap import OverlapExecutor, gpt_overlapped_forward_backward

        if self.st.dims.pp > 1 or len(self.models) != 1:
            raise ValueError("--overlap-moe-expert-parallel-comm needs pipeline size 1")
        if self.forward_step != self._default_forward_step:
            raise ValueError("--overlap-moe-expert-parallel-comm covers the language-model forward step")
        model = self.models[0]
        nmb = self.mb_calc.num_microbatches
        if not hasattr(self, "_a2a_executor"):
            self._a2a_executor = OverlapExecutor()
        self._a2a_executor.trace.clear()
        ctx = model.no_sync()
        ctx.__enter__()
        state = {"open": True}

        def leave_no_sync():
            if state["open"]:
                state["open"] = False
                ctx.__exit__(None, None, None)

        try:
            batches = (self._microbatch_inputs(self.get_batch(data_iterator)) for _ in range(nmb))
            return gpt_overlapped_forward_backward(model.module, batches, leave_no_sync, self._a2a_executor)
        finally:
            leave_no_sync()

    # ------------------------------------------------------------------ step
    def train_step(self, data_iterator) -> Dict[str, float]:
        """zero grads -> forward/backward over the micro-batches -> optimizer step -> reduce metrics."""
        t = self.tcfg
        for m in self.models:
            m.train()
        self.mb_calc.update(self.consumed_samples)  # batch-size ramp-up: micro-batches per step may grow
        self.optimizer.zero_grad()
        if t.dp_balance and self.st.dp_size > 1 and not getattr(self, "_already_balanced", False):
            data_iterator = self._balanced(data_iterator)
        # auxiliary losses (MoE balancing, MTP, indexer) are per-micro-batch means: weight each by 1 / micro-batches so
        # that, after the data-parallel average, they enter the step like the main loss does
        from ..models.moe import AuxLossScaler
        AuxLossScaler.scale = 1.0 / self.mb_calc.num_microbatches
        fb = schedules.get_forward_backward_func()
        T = t.seq_length * t.micro_batch_size
        sp_div = self.st.dims.tp if self.mcfg.sequence_parallel else 1
        def forward_backward(it):
            if t.chunkpipe_chunks and t.chunkpipe_chunks > 1:
                return self._chunkpipe_microbatches(it)
            if t.overlap_moe_expert_parallel_comm:
                return self._a2a_overlap_microbatches(it)
            return fb(forward_step_func=self.forward_step, data_iterator=it,
                      model=self.models if len(self.models) > 1 else self.models[0],
                      num_microbatches=self.mb_calc.num_microbatches,
                      tensor_shape=(T // sp_div // self.st.dims.cp, self.mcfg.hidden_size *
                                    (self.mcfg.num_residual_streams if self.mcfg.enable_hyper_connections else 1)),
                      dtype=self.mcfg.params_dtype)

        skip_update = False
        self.timers("forward-backward", 1).start()
        if self.rerun.mode == "disabled" and self.injector is None:
            reports = forward_backward(data_iterator)
        else:
            reports, skip_update = self._validated_forward_backward(forward_backward, data_iterator)
        self.timers("forward-backward", 1).stop()
        if skip_update:
            for m in self.models:
                m.finish_grad_sync()  # nothing may stay in flight when the buffers are cleared
            self.optimizer.zero_grad()
            ok, grad_norm = False, float("nan")
        else:
            self._before_optimizer_step()
            self.timers("optimizer", 1).start()
            # finishes the (possibly overlapped) data-parallel reduction first, then runs the post-sync hooks:
            # tensor-parallel partial gradients, shared embeddings
            ok, grad_norm, _ = self.optimizer.step()
            self.timers("optimizer", 1).stop()
        self._check_kernel_status()
        if ok:
            self.scheduler.step(1)
            skipped = 0
        else:
            skipped = 1
        self.iteration += 1
        self.consumed_samples += self.mb_calc.current_gbs
        metrics: Dict[str, float] = {"grad_norm": grad_norm, "skipped": skipped}
        # loss: average over micro-batches, then over the data-parallel group (last stage only)
        self.timers("loss-reduce", 2).start()
        if reports:
            keys = [k for k in reports[0] if k != "num_tokens"]
            vals = torch.stack([torch.stack([r[k].float() for r in reports]).mean() for k in keys])
            if self.st.size("dp_cp") > 1:
                dist.all_reduce(vals, group=self.st.group("dp_cp"))
                vals /= self.st.size("dp_cp")
            for k, v in zip(keys, vals.tolist()):
                metrics[k] = v
        self.timers("loss-reduce", 2).stop()
        return metrics

    # ------------------------------------------------------------------ data and evaluation
    def build_data_iterator(self, args):
        """Training stream from ``--data-path`` (one ``.bin/.idx`` prefix or weight / prefix pairs, split by
        ``--split``) or from ``--train-data-path`` with ``--valid-data-path`` beside it; also prepares ``self.valid_iterator`` when evaluation is requested. None = no data path
        (the caller falls back to synthetic data)."""
        separate = getattr(args, "train_data_path", None)
        if not (getattr(args, "data_path", None) or separate):
            return None
        from ..data.indexed_dataset import build_gpt_datasets, gpt_batch_iterator

        t, st = self.tcfg, self.st
        n_train = t.train_iters * t.global_batch_size
        n_eval = (t.train_iters // t.eval_interval + 1) * t.eval_iters * t.global_batch_size if t.eval_interval else 0
        eod = getattr(args, "eod_token_id", None)
        mask_eod = bool(getattr(args, "eod_mask_loss", False))
        if separate:  # --train-data-path / --valid-data-path: every split has data of its own, used whole
            train, _, _ = build_gpt_datasets(separate, "100,0,0", t.seq_length, (n_train, 0, 0), t.seed, eod, mask_eod)
            valid = None
            if getattr(args, "valid_data_path", None) and n_eval:
                valid, _, _ = build_gpt_datasets(args.valid_data_path, "100,0,0", t.seq_length, (n_eval, 0, 0), t.seed + 1, eod, mask_eod)
        else:
            train, valid, _ = build_gpt_datasets(args.data_path, getattr(args, "split", "949,50,1") or "949,50,1",
                                                  t.seq_length, (n_train, n_eval, 0), t.seed, eod, mask_eod)
        if train is None:
            raise ValueError("the training split of --data-path holds no documents")
        pin = self.device.type == "cuda"
        kw = dict(dp_rank=st.dp_rank, dp_size=st.dp_size, pin_memory=pin)
        self.valid_iterator = gpt_batch_iterator(valid, t.micro_batch_size, **kw) if valid is not None else None
        return gpt_batch_iterator(train, t.micro_batch_size, start_sample=self.consumed_samples, **kw)

    @torch.no_grad()
    def evaluate(self, data_iterator, iters: Optional[int] = None) -> Dict[str, float]:
        """Forward-only passes over `iters` global batches; returns the mean of every reported loss (and its
        perplexity), averaged over the data-parallel group and made known to every rank."""
        t = self.tcfg
        iters = iters or t.eval_iters or 1
        for m in self.models:
            m.eval()
        fb = schedules.get_forward_backward_func()
        T = t.seq_length * t.micro_batch_size
        sp_div = self.st.dims.tp if self.mcfg.sequence_parallel else 1
        sums: Dict[str, float] = {}
        n = 0
        for _ in range(iters):
            reports = fb(forward_step_func=self.forward_step, data_iterator=data_iterator,
                         model=self.models if len(self.models) > 1 else self.models[0],
                         num_microbatches=self.mb_calc.num_microbatches, forward_only=True,
                         tensor_shape=(T // sp_div // self.st.dims.cp, self.mcfg.hidden_size *
                                       (self.mcfg.num_residual_streams if self.mcfg.enable_hyper_connections else 1)),
                         dtype=self.mcfg.params_dtype)
            for r in reports:
                for k, v in r.items():
                    if k != "num_tokens":
                        sums[k] = sums.get(k, 0.0) + float(v)
                n += 1
        for m in self.models:
            m.train()
        keys = sorted(sums) or ["lm loss"]
        v = torch.tensor([sums.get(k, 0.0) for k in keys] + [float(n)], dtype=torch.float64, device=self.device)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(v)  # only the last pipeline stage contributes
        cnt = max(v[-1].item(), 1.0)
        out = {k: v[i].item() / cnt for i, k in enumerate(keys)}
        if "lm loss" in out:
            out["lm loss PPL"] = math.exp(min(20.0, out["lm loss"]))
        return out

    def format_eval_log(self, metrics: Dict[str, float], label: str = "validation") -> str:
        line = f" {label} loss at iteration {self.iteration} |"
        for k, v in metrics.items():
            line += (f" {k}: {v:.6E} |" if k.endswith("PPL") else f" {k} value: {v:.6E} |")
        bar = "-" * (len(line) + 1)
        return f"{bar}\n{line}\n{bar}"

    # ------------------------------------------------------------------ result validation (rerun state machine)
    def _global_loss(self, reports) -> float:
        """The step's loss as every rank must see it to take the same decision: mean over the micro-batches of all
        data-parallel ranks; NaN / Inf anywhere wins."""
        v = torch.zeros(4, dtype=torch.float64, device=self.device)  # sum, count, any nan, any inf
        for r in reports:
            x = float(r["lm loss"]) if "lm loss" in r else None
            if x is None:
                continue
            if math.isnan(x):
                v[2] += 1
            elif math.isinf(x):
                v[3] += 1
            else:
                v[0] += x
                v[1] += 1
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(v)
        s_, n, nan, inf = v.tolist()
        if nan:
            return float("nan")
        if inf:
            return float("inf")
        return s_ / max(n, 1.0)

    def _validated_forward_backward(self, forward_backward, data_iterator):
        """Forward/backward under the rerun state machine: a NaN / Inf / spiky loss triggers ONE replay of the same
        micro-batches with the same RNG state before any update is applied. A different result means a transient fault
        (the step is skipped), the same bad result a persistent one (checkpoint and exit). Returns (reports,
        skip_update)."""
        from ..ckpt.checkpointing import get_rng_state, set_rng_state

        replay = _ReplayIterator(data_iterator)
        rng = get_rng_state()
        replaying = False
        while True:
            reports = forward_backward(replay)
            loss = self._global_loss(reports)
            if self.injector is not None:
                loss = self.injector.maybe_corrupt(loss, replay=replaying)
            d = self.rerun.validate(loss)
            if d.action == "rerun":
                replaying = True
                for m in self.models:
                    m.finish_grad_sync()  # an overlapped reduction must not be running while the buffers are cleared
                self.optimizer.zero_grad()
                replay.rewind()
                set_rng_state(rng)
                continue
            if d.action == "exit":
                self.exit_requested = d.reason
            return reports, d.action in ("skip", "exit")

    def check_weight_hash_across_dp_replicas(self) -> bool:
        """Data-parallel replicas must hold bit-identical parameters: compares a checksum of every replica's parameter
        buffers over the data-parallel group (reference: loongforge/train/training_utils.py:2640-2645)."""
        if hasattr(self.optimizer, "wait_param_gather"):
            self.optimizer.wait_param_gather()  # queued (overlapped) parameter all-gathers must have landed
        acc = torch.zeros(1, dtype=torch.int64, device=self.device)
        for m in self.models:
            for buf in m._all_buffers:
                if buf.dp_group is not self.st.group("dp_cp"):
                    continue  # expert buffers are replicated over a different group
                bits = buf.param_data.view(torch.int16 if buf.param_data.element_size() == 2 else torch.int32)
                acc += bits.to(torch.int64).sum()
        lo, hi = acc.clone(), acc.clone()
        g = self.st.group("dp_cp")
        if g is not None:
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=g)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=g)
        return bool((lo == hi).item())

    def _balanced(self, data_iterator):
        """One balancing wrapper per source iterator (it buffers the step's micro-batches)."""
        cache = self.__dict__.setdefault("_balanced_iterators", {})
        w = cache.get(id(data_iterator))
        if w is None:
            from ..data.dp_balance import BalancedMicrobatchIterator
            w = cache[id(data_iterator)] = BalancedMicrobatchIterator(
                data_iterator, self.mb_calc.num_microbatches, self.st.group("dp"))
        return w

    def _chunkpipe_microbatches(self, data_iterator) -> List[dict]:
        """Sequence-chunk pipelining instead of whole-sequence micro-batches: each sequence is cut into
        ``chunkpipe_chunks`` chunks whose activations live one at a time (long-context training on one stage).
        Gradient reduction starts only after the last chunk of the last micro-batch (every chunk's backward adds to
        every parameter), i.e. in the optimizer's ``finish_grad_sync``."""
        from .chunkpipe import gpt_chunkpipe_step

        t, st = self.tcfg, self.st
        if st.dims.cp > 1 or t.micro_batch_size != 1 or len(self.models) != 1:
            raise ValueError("chunk pipelining needs cp = 1, micro batch size 1 and no virtual pipeline stages")
        model = self.models[0]
        nmb = self.mb_calc.num_microbatches
        reports = []
        with model.no_sync():
            for _ in range(nmb):
                b = self.get_batch(data_iterator)
                mask = b["loss_mask"].reshape(-1)
                n_valid = b.get("num_valid_tokens") or int(mask.numel())
                scale = 1.0 / (max(n_valid, 1) * nmb)
                loss = gpt_chunkpipe_step(model.module, b["tokens"].reshape(-1), b["position_ids"].reshape(-1),
                                          b["labels"].reshape(-1), mask, t.chunkpipe_chunks, scale)
                if st.is_last_stage:
                    reports.append({"lm loss": loss * nmb, "num_tokens": n_valid})
        return reports

    def _allreduce_embedding_grads(self):
        """Sum the word-embedding gradients of the first and last pipeline stage (tied output layer and / or
        multi-token prediction). Both copies sit alone in identically laid out buffers, so after a sharded
        data-parallel reduction each rank's valid slice pairs with the same slice on the other stage."""
        g = self.st.group("embd")
        for p in self._shared_embeddings:
            dist.all_reduce(p.main_grad, group=g)

    def _before_optimizer_step(self):
        """Hook between the last backward and the optimizer step (subclasses: encoder backward of the
        heterogeneous-DP schedule)."""

    def _check_kernel_status(self):
        """Read the native kernels' status word once per step and raise on the first wait that gave up, on every
        rank of the job at the same step: a fused kernel whose peer wait ran out has returned partly written
        outputs, so the step must not be trusted."""
        if self.device.type != "cuda":
            return
        from ..ops import _ext
        if not _ext.available():
            return
        word = _ext.status_tensor(self.device)
        code = word.clone()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(code, op=dist.ReduceOp.MAX)
        c = int(code.item())
        if c != 0:
            word.zero_()
            raise RuntimeError(f"iteration {self.iteration}: native kernel error {c} on some rank: "
                               f"{_ext.STATUS_NAMES.get(c, 'unknown')}")

    def _allreduce_sequence_parallel_grads(self):
        """Replicated parameters whose gradient is only a PARTIAL sum on each TP rank are summed over the TP group:
        norm weights that see a sequence shard (sequence parallelism), and per-head norm weights applied to this
        rank's heads only (``tp_partial_grad``: QK layernorm, gated-delta-net output norm). Runs as the first
        post-sync hook of the optimizer, i.e. after the data-parallel reduction. With the sharded optimizer only this
        rank's shard of each gradient is valid by then; TP peers hold the same shard, so summing whole tensors is
        still right where it matters."""
        self.timers("partial-grads-all-reduce", 2).start()
        try:
            st = self.st
            if st.dims.tp == 1:
                return
            sp = self.mcfg.sequence_parallel
            grads = []
            for m in self.models:
                for p in m.module.parameters():
                    if p.requires_grad and ((sp and getattr(p, "sequence_parallel", False))
                                            or getattr(p, "tp_partial_grad", False)):
                        grads.append(p.main_grad)
            if not grads:
                return
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, group=st.group("tp"))
            off = 0
            for g in grads:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g))
                off += n
        finally:
            self.timers("partial-grads-all-reduce", 2).stop()

    # ------------------------------------------------------------------ logging
    def flops_per_step(self) -> float:
        return self.mcfg.flops_per_token(self.tcfg.seq_length) * self.tcfg.seq_length * self.mb_calc.current_gbs

    def format_log(self, metrics: Dict[str, float], elapsed_ms: float, peak_tflops: Optional[float] = None) -> str:
        """The reference's log line (loongforge/train/training_utils.py:2278-2394), parsed by
        tests/llm_vlm/tools/log2json.py:19-29."""
        t = self.tcfg
        tokens = t.seq_length * self.mb_calc.current_gbs
        tps = tokens / (elapsed_ms / 1e3) / self.world
        s = " [%s] iteration %8d/%8d |" % (time.strftime("%Y-%m-%d %H:%M:%S"), self.iteration, t.train_iters)
        s += " consumed samples: %12d |" % self.consumed_samples
        s += " elapsed time per iteration (ms): %.1f |" % elapsed_ms
        s += " throughput (token/sec/GPU): %.1f |" % tps
        if t.log_throughput:
            tf = self.flops_per_step() / (elapsed_ms / 1e3) / 1e12 / self.world
            s += " flop throughput (TFLOP/sec/GPU): %.1f |" % tf
        s += " learning rate: %.6E |" % self.optimizer.param_groups[0]["lr"]
        s += " global batch size: %5d |" % self.mb_calc.current_gbs
        for k, v in metrics.items():
            if k in ("grad_norm", "skipped"):
                continue
            s += " %s: %.6E |" % (k, v)
        s += " loss scale: %.1f |" % 1.0
        s += " grad norm: %.6f |" % metrics.get("grad_norm", float("nan"))
        s += " number of skipped iterations: %3d |" % metrics.get("skipped", 0)
        s += " number of nan iterations: %3d |" % self._nan
        if self.device.type == "cuda":
            s += " mem-allocated-bytes-avg(MB): %.1f |" % (torch.cuda.memory_allocated() / 2 ** 20)
            s += " mem-max-allocated-bytes-avg(MB): %.1f |" % (torch.cuda.max_memory_allocated() / 2 ** 20)
        return s

    # ------------------------------------------------------------------ loop
    def train(self, data_iterator, *, on_log: Optional[Callable[[str], None]] = None) -> List[Dict[str, float]]:
        t = self.tcfg
        history = []
        is_log_rank = (not dist.is_initialized()) or dist.get_rank() == dist.get_world_size() - 1
        skip = set(t.iterations_to_skip or ())
        while self.iteration < t.train_iters:
            if (self.iteration + 1) in skip:
                # the iteration's data is consumed so that later iterations see what they would have seen
                self.mb_calc.update(self.consumed_samples)
                for _ in range(self.mb_calc.num_microbatches):
                    next(data_iterator)
                self.iteration += 1
                self.consumed_samples += self.mb_calc.current_gbs
                continue
            t0 = self._now()
            metrics = self.train_step(data_iterator)
            if t.check_weight_hash_interval and self.iteration % t.check_weight_hash_interval == 0:
                if not self.check_weight_hash_across_dp_replicas():
                    raise RuntimeError(f"parameters differ between data-parallel replicas at iteration {self.iteration}")
            elapsed_ms = (self._now() - t0) * 1e3
            self.num_flops_so_far += self.flops_per_step()
            history.append(metrics)
            if t.check_for_nan_in_loss and "lm loss" in metrics and not math.isfinite(metrics["lm loss"]):
                self._nan += 1
                if t.exit_on_nan:
                    raise RuntimeError(f"non-finite loss at iteration {self.iteration}")
            if self.iteration % t.log_interval == 0:
                line = self.format_log(metrics, elapsed_ms)
                if is_log_rank:
                    (on_log or print)(line)
                if self.timers.timers:  # --timing-log-level >= 1: per-phase times, min and max over the ranks
                    if t.log_timers_to_tensorboard:
                        for name, tm in self.timers.timers.items():
                            metrics[f"timers/{name}-ms"] = tm.elapsed(reset=False) * 1e3 / t.log_interval
                    report = self.timers.report(normalizer=float(t.log_interval))
                    if is_log_rank:
                        (on_log or print)(report)
            if (t.eval_interval and t.eval_iters and self.iteration % t.eval_interval == 0
                    and getattr(self, "valid_iterator", None) is not None):
                ev = self.evaluate(self.valid_iterator)
                self.last_eval = ev
                if is_log_rank:
                    (on_log or print)(self.format_eval_log(ev))
            if t.save and t.save_interval and self.iteration % t.save_interval == 0:
                self.save_checkpoint(t.save)
            stop = self.exit_requested
            for h in getattr(self, "hooks", ()):
                stop = h.on_step_end(self, metrics, elapsed_ms) or stop
            if stop:
                # a hook asked for checkpoint-and-exit (signal, time limit, exit interval)
                if t.save:
                    self.save_checkpoint(t.save)
                break
        if hasattr(self.optimizer, "wait_param_gather"):
            self.optimizer.wait_param_gather()  # whoever reads the parameters next (export, evaluation code) sees them whole
        for h in getattr(self, "hooks", ()):
            h.on_train_end(self)
        if getattr(self, "_pending_save", None) is not None:
            from ..ckpt import checkpointing
            checkpointing.finalize_async_save(self)
        return history

    def _now(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        return time.perf_counter()

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, path: str):
        from ..ckpt import checkpointing
        if hasattr(self.optimizer, "wait_param_gather"):
            self.optimizer.wait_param_gather()  # parameters are read outside a forward pass
        checkpointing.save_checkpoint(path, self)

    def load_checkpoint(self, path: str, **kw):
        from ..ckpt import checkpointing
        return checkpointing.load_checkpoint(path, self, **kw)


class _ReplayIterator:
    """Remembers what the current step pulled from the data iterator so that the step can be replayed."""

    def __init__(self, it):
        self.it, self.seen, self.pos = it, [], 0

    def __iter__(self):
        return self

    def __next__(self):
        if self.pos < len(self.seen):
            item = self.seen[self.pos]
        else:
            item = next(self.it)
            self.seen.append(item)
        self.pos += 1
        return item

    def rewind(self):
        self.pos = 0
