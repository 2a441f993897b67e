"""Consistency checks and derived settings of a training run (the rules the reference enforces in
loongforge/train/validators.py:140-620 and through Megatron's ``validate_args``)."""
from __future__ import annotations

import os


def validate(args, cfg, tc, dims) -> None:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    mp = dims.tp * dims.pp * dims.cp
    if world % mp:
        raise ValueError(f"world size {world} is not divisible by tp*pp*cp = {mp}")
    dp = world // mp
    if tc.global_batch_size % (tc.micro_batch_size * dp):
        raise ValueError(f"global batch size {tc.global_batch_size} must be a multiple of micro batch size x data "
                         f"parallel size ({tc.micro_batch_size} x {dp})")
    if cfg.sequence_parallel and dims.tp == 1:
        cfg.sequence_parallel = False  # Megatron silently disables SP without TP
    if cfg.tp_comm_overlap and not cfg.sequence_parallel:
        raise ValueError("--tp-comm-overlap needs --sequence-parallel")
    if getattr(args, "fp16", False) and cfg.tp_comm_overlap:
        cfg.tp_comm_overlap = False  # reference: forced off for fp16 (validators.py:436-443)
    if cfg.num_attention_heads % dims.tp or cfg.num_query_groups % dims.tp:
        raise ValueError("attention heads / query groups must divide by the tensor parallel size")
    if dims.cp > 1 and tc.seq_length % (2 * dims.cp):
        raise ValueError("sequence length must divide by 2 x context parallel size")
    if cfg.sequence_parallel and (tc.seq_length * tc.micro_batch_size // dims.cp) % dims.tp:
        raise ValueError("tokens per micro-batch must divide by tp under sequence parallelism")
    if cfg.num_moe_experts:
        if cfg.num_moe_experts % dims.ep:
            raise ValueError("number of experts must divide by the expert parallel size")
        stage = dims.tp * dims.cp * dp
        if stage % (dims.ep * dims.etp):
            raise ValueError("tp*cp*dp must divide by ep*etp")
    elif dims.ep > 1:
        raise ValueError("--expert-model-parallel-size > 1 needs an MoE model")
    # Ulysses degree maps onto the a2a (or hierarchical) context-parallel communication type
    u = getattr(args, "context_parallel_ulysses_degree", None)
    if u:
        if dims.cp % u:
            raise ValueError("context parallel size must divide by the Ulysses degree")
        args.cp_comm_type = "a2a" if u == dims.cp else "a2a+p2p"
    if getattr(args, "enable_full_hetero_dp", False) and dims.cp > 1:
        raise ValueError("full heterogeneous DP does not support context parallelism")
    if getattr(args, "enable_encoder_hetero_dp", False) and (args.encoder_tensor_model_parallel_size or 1) != 1:
        raise ValueError("encoder hetero-DP needs encoder tensor parallel size 1")
    if getattr(args, "enable_chunkpipe", False) and not getattr(args, "chunksize", None):
        raise ValueError("--enable-chunkpipe needs --chunksize")
    if tc.training_phase == "sft" and not (getattr(args, "sft_dataset", None) or getattr(args, "mock_data", False)
                                           or getattr(args, "data_path", None) or getattr(args, "train_data_path", None)):
        raise ValueError("SFT needs --sft-dataset / --data-path (or --mock-data)")
    if dims.vpp and dims.vpp > 1 and cfg.num_layers % (dims.pp * dims.vpp) and not tc.custom_pipeline_layers:
        raise ValueError("num_layers must divide by pp x virtual stages")
    if dims.pp > 1 and cfg.num_layers % dims.pp and not tc.custom_pipeline_layers \
            and not getattr(args, "pipeline_model_parallel_layout", None):
        raise ValueError(f"{cfg.num_layers} layers do not divide by pipeline size {dims.pp}: give --custom-pipeline-layers")
    _validate_sft(args, tc)
    _validate_attention_variants(args, cfg, tc, dims)
    _validate_moe(args, cfg, tc, dims)
    _validate_multimodal(args, cfg, tc, dims)


def _validate_sft(args, tc) -> None:
    """Supervised fine-tuning rules (reference: loongforge/train/validators.py:140-312)."""
    if tc.training_phase != "sft":
        return
    if getattr(args, "train_on_prompt", False) and getattr(args, "history_mask_loss", False):
        raise ValueError("--train-on-prompt and --history-mask-loss cannot both be set")
    if getattr(args, "sft_data_streaming", False) and getattr(args, "sft_sort_batch", False):
        raise ValueError("--sft-sort-batch cannot be used together with --sft-data-streaming")
    if getattr(args, "packing_sft_data", False) and tc.micro_batch_size > 1:
        raise ValueError("--packing-sft-data packs one row per micro-batch: use --micro-batch-size 1")
    tmpl = getattr(args, "chat_template", None)
    if tmpl:
        from ..data.chat_template import get_template
        get_template(tmpl)  # unknown names fail here, not after the model is built
    if getattr(args, "sft_dataset", None) and getattr(args, "tokenizer_type", None) not in (None, "HFTokenizer", "NullTokenizer"):
        raise ValueError("--tokenizer-type should be HFTokenizer when the training phase is sft")


def _validate_attention_variants(args, cfg, tc, dims) -> None:
    """Sparse attention / chunk pipelining / overlap-schedule combinations (reference: validators.py:314-366)."""
    if getattr(args, "use_dsa_sp_first", False) or getattr(cfg, "dsa_sp_first", False):
        if not cfg.sequence_parallel:
            raise ValueError("--use-dsa-sp-first requires --sequence-parallel")
        if not getattr(cfg, "use_dsa", False):
            raise ValueError("--use-dsa-sp-first requires the sparse attention variant (--use-dsa-fused)")
        if dims.cp > 1:
            raise ValueError("--use-dsa-sp-first does not combine with context parallelism")
    share = getattr(cfg, "dsa_indexer_topk_freq", 1) or 1
    if share > 1 and not getattr(cfg, "use_dsa", False):
        raise ValueError("--dsa-indexer-topk-freq > 1 (IndexShare) requires the sparse attention variant")
    if tc.overlap_moe_expert_parallel_comm:
        if dims.pp > 1:
            raise ValueError("--overlap-moe-expert-parallel-comm needs pipeline size 1")
        if not cfg.num_moe_experts:
            raise ValueError("--overlap-moe-expert-parallel-comm needs an MoE model")
        if cfg.recompute_granularity == "full":
            raise ValueError("--overlap-moe-expert-parallel-comm does not cover full activation recomputation")
        world = int(os.environ.get("WORLD_SIZE", "1"))
        dp = world // (dims.tp * dims.pp * dims.cp)
        if tc.global_batch_size // (tc.micro_batch_size * max(dp, 1)) < 2:
            raise ValueError("--overlap-moe-expert-parallel-comm interleaves micro-batches: at least two per step are needed")
    if tc.chunkpipe_chunks and tc.chunkpipe_chunks > 1:
        if dims.cp > 1 or tc.micro_batch_size != 1 or (dims.vpp or 1) > 1:
            raise ValueError("chunk pipelining needs cp = 1, micro batch size 1 and no virtual pipeline stages")
        if tc.seq_length % tc.chunkpipe_chunks:
            raise ValueError("--seq-length must divide by the number of chunks (seq-length / chunksize)")


def _validate_moe(args, cfg, tc, dims) -> None:
    if not cfg.num_moe_experts:
        # dispatcher types that only exist for MoE models fall back, as the reference does (validators.py:359-365)
        if getattr(args, "moe_token_dispatcher_type", None) in ("allgather", "alltoall_seq"):
            args.moe_token_dispatcher_type = "alltoall"
        return
    if cfg.moe_router_topk > cfg.num_moe_experts:
        raise ValueError("--moe-router-topk exceeds the number of experts")
    g, gk = cfg.moe_router_num_groups, cfg.moe_router_group_topk
    if g:
        if cfg.num_moe_experts % g:
            raise ValueError("number of experts must divide by --moe-router-num-groups")
        if gk and (gk > g or cfg.moe_router_topk > gk * (cfg.num_moe_experts // g)):
            raise ValueError("--moe-router-group-topk groups cannot hold --moe-router-topk experts")
    if cfg.moe_token_dispatcher_type == "peer" and dims.etp > 1:
        raise ValueError("the peer-memory dispatcher does not cover expert tensor parallelism; use alltoall")


def _validate_multimodal(args, cfg, tc, dims) -> None:
    """Vision-language and diffusion rules (reference: validators.py:370-420 and the WAN trainers' shape checks)."""
    mtl = getattr(args, "max_text_length", None)
    if mtl and dims.cp > 1 and mtl % dims.cp:
        args.max_text_length = (mtl + dims.cp - 1) // dims.cp * dims.cp  # text length divisible by the CP size
    enc_tp = getattr(args, "encoder_tensor_model_parallel_size", None)
    if enc_tp and dims.tp % enc_tp:
        raise ValueError("the decoder's tensor parallel size must divide by the encoder's")
    if getattr(args, "enable_full_hetero_dp", False) and getattr(args, "enable_encoder_hetero_dp", False):
        raise ValueError("--enable-full-hetero-dp replaces --enable-encoder-hetero-dp: give one of them")
    name = str(getattr(args, "model_name", "") or "")
    if name.startswith("wan"):
        # WAN latents: 4x temporal / 8x spatial VAE compression, then (1, 2, 2) patches; Ulysses splits the token axis
        frames = getattr(args, "num_frames", None) or getattr(args, "frame_num", None)
        if frames and (int(frames) - 1) % 4:
            raise ValueError("WAN video lengths must be 4 k + 1 frames")
        for side in ("height", "width"):
            v = getattr(args, side, None)
            if v and int(v) % 16:
                raise ValueError(f"WAN {side} must be a multiple of 16 (8x VAE, 2x patch)")


# Flags that are accepted for command-line compatibility but whose feature is reached through a library entry point
# rather than the training CLI today. Nothing is ignored silently: `unwired_flag_notes` lists what was requested.
_LIBRARY_ONLY = {
    "enable_cuda_graph": "CUDA graphs: runtime.cuda_graphs.GraphedCallable / embodied.cuda_graph.MicrobatchGraphRunner",
}


# Flags of the reference that configure a library this framework does not contain, or select between alternatives of
# which only one exists here. They are accepted so that the reference's launch scripts run unchanged; when one is given,
# the note says what happens instead.
_ACCEPTED = {
    "absorb_backend": "the MLA absorb products use one einsum formulation",
    "moe_permute_fusion": "token permutation is always fused into the dispatch path",
    "delay_wgrad_compute": "weight gradients are computed with their data gradients",
    "use_precision_aware_optimizer": "moment precision is chosen with --exp-avg-dtype / --exp-avg-sq-dtype",
    "fp8_param_gather": "parameters are gathered in bf16",
    "cross_entropy_fusion_impl": "one fused linear + cross-entropy implementation exists",
    "use_flash_attn": "attention always runs on the in-tree flash kernel on GPUs",
    "cuda_graph_scope": "graph capture is offered by runtime.cuda_graphs for callables, not selected by scope",
    "tokenizer_model": "tokenizers load from --hf-tokenizer-path",
    "dataloader_type": "one cyclic, resumable sampler is used",
    "variable_seq_lengths": "pipeline stages exchange fixed-shape activations; packed rows are padded to --seq-length",
    "dist_ckpt_strictness": "unexpected or missing checkpoint keys raise",
    "detail_log_interval": "one log interval exists",
}


def unwired_flag_notes(args) -> list:
    notes = []
    from .arguments import build_parser
    parser = build_parser()
    for flag, what in _ACCEPTED.items():
        v = getattr(args, flag, None)
        if v not in (None, False, 0, "", []) and v != parser.get_default(flag):  # only what the user actually set
            notes.append(f"--{flag.replace('_', '-')} was given: {what}")
    for flag, where in _LIBRARY_ONLY.items():
        v = getattr(args, flag, None)
        if v:
            notes.append(f"--{flag.replace('_', '-')} was given: not selectable from this CLI yet; available as {where}")
    return notes


def apply_aliases(args) -> None:
    """Reference flags that select a feature this framework provides under another name."""
    if getattr(args, "moe_enable_deepep", False) and getattr(args, "moe_token_dispatcher_type", None) in (None, "alltoall", "flex"):
        # DeepEP's role (dispatch / combine kernels over NVLink) is played by the peer-memory dispatcher
        args.moe_token_dispatcher_type = "peer"
