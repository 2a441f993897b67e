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
    if tc.training_phase == "sft" and not (getattr(args, "sft_dataset", None) or getattr(args, "mock_data", False)):
        raise ValueError("SFT needs --sft-dataset (or --mock-data)")
    if dims.vpp and dims.vpp > 1 and cfg.num_layers % (dims.pp * dims.vpp) and not tc.custom_pipeline_layers:
        raise ValueError("num_layers must divide by pp x virtual stages")


# Flags that are accepted for command-line compatibility but whose feature is reached through a library entry point
# rather than the training CLI today. Nothing is ignored silently: `unwired_flag_notes` lists what was requested.
_LIBRARY_ONLY = {
    "enable_cuda_graph": "CUDA graphs: runtime.cuda_graphs.GraphedCallable / embodied.cuda_graph.MicrobatchGraphRunner",
}


# Flags of the reference that configure a library this framework does not contain, or select between alternatives of
# which only one exists here. They are accepted so that the reference's launch scripts run unchanged; when one is given,
# the note says what happens instead.
_ACCEPTED = {
    "use_dsa_sp_first": "sparse attention runs head-parallel under TP with a replicated indexer; there is no separate sequence-first mode",
    "absorb_backend": "the MLA absorb products use one einsum formulation",
    "moe_permute_fusion": "token permutation is always fused into the dispatch path",
    "delay_wgrad_compute": "weight gradients are computed with their data gradients",
    "use_precision_aware_optimizer": "moment precision is chosen with --exp-avg-dtype / --exp-avg-sq-dtype",
    "fp8_param_gather": "parameters are gathered in bf16",
    "cross_entropy_fusion_impl": "one fused linear + cross-entropy implementation exists",
    "use_flash_attn": "attention always runs on the in-tree flash kernel on GPUs",
    "cuda_graph_scope": "graph capture is offered by runtime.cuda_graphs for callables, not selected by scope",
    "tokenizer_model": "tokenizers load from --hf-tokenizer-path",
    "sft_dataset_config": "dataset options are given as flags",
    "sft_data_streaming": "SFT datasets are read eagerly",
    "dataloader_type": "one cyclic, resumable sampler is used",
    "num_workers": "batches are assembled in the training process",
    "variable_seq_lengths": "pipeline stages exchange fixed-shape activations; packed rows are padded to --seq-length",
    "dist_ckpt_strictness": "unexpected or missing checkpoint keys raise",
    "detail_log_interval": "one log interval exists",
    "wandb_exp_name": "the run name is the output directory",
    "packing_batch_size": "the online packer's buffer holds 16 samples (64 for SFT text)",
    "frame_num": "video inputs are not decoded by the built-in loaders (image-text shards only)",
    "fps": "video inputs are not decoded by the built-in loaders (image-text shards only)",
}


def unwired_flag_notes(args) -> list:
    notes = []
    for flag, what in _ACCEPTED.items():
        v = getattr(args, flag, None)
        if v not in (None, False, 0, "", []):
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
