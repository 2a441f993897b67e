"""Model configuration dataclasses.

One flat ``TransformerConfig`` covers dense, MoE, MLA/DSA and vision stacks; family presets
(``models/registry.py``) and YAML files fill it. Field names follow Megatron's
``TransformerConfig`` / ``MLATransformerConfig`` (the reference builds these from args in
loongforge/models/utils.py:108-176 and loongforge/models/common/base_model_config.py:26-69), so
that the reference's YAML model files map onto it one to one.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Union

import torch


@dataclasses.dataclass
class TransformerConfig:
    # ---- architecture
    num_layers: int = 2
    hidden_size: int = 256
    num_attention_heads: int = 4
    num_query_groups: Optional[int] = None
    kv_channels: Optional[int] = None  # head dim
    ffn_hidden_size: Optional[int] = None
    vocab_size: int = 32000
    padded_vocab_size: Optional[int] = None
    make_vocab_size_divisible_by: int = 128
    max_position_embeddings: int = 8192
    normalization: str = "RMSNorm"  # or LayerNorm
    layernorm_epsilon: float = 1e-5
    layernorm_zero_centered_gamma: bool = False
    activation: str = "swiglu"  # swiglu | gelu | geglu | quick_gelu | relu | silu
    gated_linear_unit: bool = True
    add_bias_linear: bool = False
    add_qkv_bias: bool = False
    qk_layernorm: bool = False
    untie_embeddings_and_output_weights: bool = True
    position_embedding_type: str = "rope"  # rope | mrope | yarn | none | learned_absolute
    rotary_base: float = 10000.0
    rotary_percent: float = 1.0
    rotary_interleaved: bool = False
    rotary_scaling_factor: float = 1.0
    rotary_dynamic_ntk: bool = False  # enlarge the rotary base for sequences beyond max_position_embeddings
    rotary_dynamic_ntk_factor: float = 8.0
    mrope_section: Optional[List[int]] = None
    mrope_interleaved: bool = False
    attention_dropout: float = 0.0
    hidden_dropout: float = 0.0
    attention_softmax_scale: Optional[float] = None
    causal: bool = True
    window_size: Optional[int] = None
    init_method_std: float = 0.02
    output_layer_init_std: Optional[float] = None
    # ---- yarn
    yarn_scaling_factor: float = 1.0
    yarn_original_max_position: int = 4096
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    yarn_mscale: float = 1.0
    yarn_mscale_all_dim: float = 0.0
    # ---- MoE
    num_moe_experts: Optional[int] = None
    moe_router_topk: int = 2
    moe_ffn_hidden_size: Optional[int] = None
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_shared_expert_gate: bool = False  # sigmoid gate on the shared expert's output (Qwen3-Next, Qwen3.5)
    moe_layer_freq: Union[int, List[int]] = 1
    moe_router_score_function: str = "softmax"  # softmax | sigmoid
    moe_router_pre_softmax: bool = False
    moe_router_enable_expert_bias: bool = False
    moe_router_bias_update_rate: float = 1e-3
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_load_balancing_type: str = "aux_loss"  # aux_loss | seq_aux_loss | none
    moe_aux_loss_coeff: float = 0.0
    moe_z_loss_coeff: Optional[float] = None
    moe_token_dispatcher_type: str = "alltoall"  # alltoall (NCCL) | peer (NVLink peer-memory kernels, CUDA only)
    # receive-buffer rows per rank = factor * local tokens * top-k; routing of an untrained router is easily 2-3x
    # skewed, and growing the buffers later costs a collective re-allocation
    moe_peer_capacity_factor: float = 4.0
    moe_grouped_gemm: bool = True
    moe_expert_capacity_factor: Optional[float] = None
    # ---- MLA / DSA
    multi_latent_attention: bool = False
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 512
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 128
    use_dsa: bool = False
    dsa_indexer_n_heads: int = 64
    dsa_indexer_head_dim: int = 128
    dsa_indexer_topk: int = 2048
    dsa_indexer_loss_coeff: float = 0.0
    # IndexShare (GLM-5.2): only some layers own an indexer; the others reuse the latest computed top-k indices.
    # Layers below the offset and every `freq`-th layer from (offset + freq - 1) on compute their own.
    dsa_indexer_topk_freq: int = 1
    # sequence-first sparse attention under TP + SP: every rank attends from ITS tokens with ALL heads (up projections
    # and the output projection replicated); only the 576-value compressed keys and the indexer keys are gathered
    dsa_sp_first: bool = False
    dsa_indexer_skip_topk_offset: int = 0
    dsa_indexer_rope_interleaved: bool = False  # GLM-5.x rotates the indexer's rotary part in interleaved pairs
    dsa_indexer_rotate_activation: bool = True  # Hadamard transform of the indexer q / k (DeepSeek-V3.2: on, GLM-5.x: off)
    dsa_indexer_k_norm_epsilon: float = 1e-6
    # ---- hybrid attention (Qwen3-Next / Qwen3.5): per-layer "full_attention" | "linear_attention"
    layer_types: Optional[List[str]] = None
    full_attention_interval: Optional[int] = None  # every n-th layer is full attention when layer_types is unset
    attention_output_gate: bool = False
    linear_conv_kernel_dim: int = 4
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    # ---- DeepSeek-V4: compressed sparse attention, hyper-connections, hash-routed first MoE layers
    csa_compress_ratios: Optional[List[int]] = None  # per layer: 0 (window only) or the tokens folded per entry
    csa_window_size: int = 128
    enable_hyper_connections: bool = False
    num_residual_streams: int = 4
    mhc_sinkhorn_iterations: int = 20
    mhc_init_gating_factor: float = 1e-2
    moe_n_hash_layers: int = 0  # the first n MoE layers pick experts by a hash of the token id
    swiglu_limit: Optional[float] = None
    # ---- ERNIE-4.5-VL: modality-routed expert sets and 3-D rotary layout
    moe_multi_type: bool = False
    moe_vision_num_experts: Optional[int] = None
    moe_vision_ffn_hidden_size: Optional[int] = None
    rope_3d_freq_allocation: int = 0  # > 0: the last n rotary frequencies follow the temporal position
    # ---- MiniMax: QK RMSNorm over the whole projection (all heads) instead of per head
    qk_layernorm_full: bool = False
    # ---- MTP
    mtp_num_layers: int = 0
    mtp_loss_scaling_factor: float = 0.1
    mtp_hidden_first: bool = False  # MiMo: eh_proj input is [hidden, embedding] instead of [embedding, hidden]
    # ---- precision
    params_dtype: torch.dtype = torch.float32
    fp8: Optional[str] = None  # None | "blockwise"
    fp32_residual_connection: bool = False
    # ---- parallel behaviour
    sequence_parallel: bool = False
    tp_comm_overlap: bool = False  # fused all-gather->GEMM / GEMM->reduce-scatter over peer memory
    recompute_granularity: Optional[str] = None  # None | full | selective
    recompute_method: Optional[str] = None  # uniform | block
    recompute_num_layers: Optional[int] = None
    cross_entropy_loss_fusion: bool = True
    cross_entropy_chunk_tokens: int = 2048
    gradient_accumulation_fusion: bool = True
    # ---- vision specifics
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    in_channels: int = 3
    fullatt_block_indexes: Optional[List[int]] = None
    vision_window_size: int = 112
    model_family: str = "llama"

    def __post_init__(self):
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.kv_channels is None:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.ffn_hidden_size is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.activation in ("swiglu", "geglu"):
            self.gated_linear_unit = True
        if self.padded_vocab_size is None:
            self.padded_vocab_size = self.vocab_size
        if self.output_layer_init_std is None:
            self.output_layer_init_std = self.init_method_std
        if self.moe_ffn_hidden_size is None:
            self.moe_ffn_hidden_size = self.ffn_hidden_size

    # helpers ---------------------------------------------------------------------
    def layer_type(self, layer_idx: int) -> str:
        if self.layer_types is not None:
            return self.layer_types[layer_idx]
        if self.full_attention_interval:
            return "full_attention" if (layer_idx + 1) % self.full_attention_interval == 0 else "linear_attention"
        return "full_attention"

    def pad_vocab(self, tp: int) -> int:
        mult = self.make_vocab_size_divisible_by * tp
        self.padded_vocab_size = ((self.vocab_size + mult - 1) // mult) * mult
        return self.padded_vocab_size

    def dsa_computes_topk(self, layer_idx: int) -> bool:
        """Does this (0-based) layer own an indexer, or does it reuse another layer's top-k (IndexShare)?"""
        f, off = self.dsa_indexer_topk_freq, self.dsa_indexer_skip_topk_offset
        if f <= 1 or layer_idx < off or layer_idx >= self.num_layers:  # MTP layers (>= num_layers) always compute
            return True
        return (layer_idx - off + 1) % f == 0

    def dsa_source_layer(self, layer_idx: int) -> int:
        """The layer whose top-k indices this layer uses (itself when it computes them)."""
        l = layer_idx
        while not self.dsa_computes_topk(l):
            l -= 1
        return l

    def is_moe_layer(self, layer_idx: int) -> bool:
        if self.num_moe_experts is None:
            return False
        f = self.moe_layer_freq
        if isinstance(f, int):
            return layer_idx % f == 0
        return bool(f[layer_idx])

    def num_parameters(self) -> int:
        """Parameter count of the full (unsharded) language model."""
        h, L = self.hidden_size, self.num_layers
        d = self.kv_channels
        if self.multi_latent_attention:
            qd = self.qk_head_dim + self.qk_pos_emb_head_dim
            nh = self.num_attention_heads
            attn = 0
            if self.q_lora_rank:
                attn += h * self.q_lora_rank + self.q_lora_rank * nh * qd + self.q_lora_rank
            else:
                attn += h * nh * qd
            attn += h * (self.kv_lora_rank + self.qk_pos_emb_head_dim) + self.kv_lora_rank
            attn += self.kv_lora_rank * nh * (self.qk_head_dim + self.v_head_dim)
            attn += nh * self.v_head_dim * h
        else:
            attn = h * (self.num_attention_heads + 2 * self.num_query_groups) * d + self.num_attention_heads * d * h
        glu = 3 if self.gated_linear_unit else 2
        total = 0
        for i in range(L):
            total += attn + 2 * h
            if self.is_moe_layer(i):
                total += self.num_moe_experts * glu * h * self.moe_ffn_hidden_size + h * self.num_moe_experts
                if self.moe_shared_expert_intermediate_size:
                    total += glu * h * self.moe_shared_expert_intermediate_size
            else:
                total += glu * h * self.ffn_hidden_size
        total += h  # final norm
        total += self.padded_vocab_size * h * (2 if self.untie_embeddings_and_output_weights else 1)
        return total

    def flops_per_token(self, seq_len: int) -> float:
        """Training (fwd+bwd) model FLOPs per token, Megatron's accounting: 6 x matmul params
        touched per token + causal attention score/value matmuls."""
        h, L = self.hidden_size, self.num_layers
        d = self.kv_channels
        glu = 3 if self.gated_linear_unit else 2
        per_tok = 0.0
        for i in range(L):
            if self.multi_latent_attention:
                nh = self.num_attention_heads
                qd = self.qk_head_dim + self.qk_pos_emb_head_dim
                lin = (h * self.q_lora_rank + self.q_lora_rank * nh * qd) if self.q_lora_rank else h * nh * qd
                lin += h * (self.kv_lora_rank + self.qk_pos_emb_head_dim)
                lin += self.kv_lora_rank * nh * (self.qk_head_dim + self.v_head_dim) + nh * self.v_head_dim * h
                kv_len = min(seq_len, self.dsa_indexer_topk) if self.use_dsa else seq_len / 2
                attn_mm = nh * (qd + self.v_head_dim) * kv_len
                if self.use_dsa:
                    attn_mm += self.dsa_indexer_n_heads * self.dsa_indexer_head_dim * seq_len / 2
            else:
                lin = h * (self.num_attention_heads + 2 * self.num_query_groups) * d + self.num_attention_heads * d * h
                attn_mm = self.num_attention_heads * 2 * d * (seq_len / 2 if self.causal else seq_len)
            if self.is_moe_layer(i):
                mlp = self.moe_router_topk * glu * h * self.moe_ffn_hidden_size + h * self.num_moe_experts
                if self.moe_shared_expert_intermediate_size:
                    mlp += glu * h * self.moe_shared_expert_intermediate_size
            else:
                mlp = glu * h * self.ffn_hidden_size
            per_tok += 6.0 * (lin + mlp) + 6.0 * attn_mm
        per_tok += 6.0 * self.padded_vocab_size * h
        return per_tok
