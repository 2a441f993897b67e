"""Vision-language composition: vision encoder -> projector -> language model, with
heterogeneous parallelism between the components.

Counterpart of the reference's ``OmniCombinationModel`` / ``OmniEncoderModel``
(loongforge/models/omni_models/omni_combination_model.py:191-597,
omni_encoder_model.py:66-218,386-397). The encoder and projector live in their own named parallel
state (``image_encoder``, typically TP=1) while the language model uses the default state (e.g.
TP2 + sequence parallel, PP2); entering the encoder switches the current state and leaving
restores it. With ``encoder_hetero_dp`` the ranks of one language-model TP group split the images
of the micro-batch among themselves (the encoder runs data parallel over the TP group) and
all-gather the projected embeddings, instead of every rank encoding every image. The encoder
exists only on the first pipeline stage. Image embeddings replace the ``image_token_id`` slots of
the text embedding sequence (masked scatter) before the sequence is scattered for sequence
parallelism.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel import mappings as M
from ..parallel import state as ps
from .config import TransformerConfig
from .gpt import GPTModel
from .vision import MLPAdapter, VisionModel

ENCODER_STATE = "image_encoder"
IGNORE_INDEX = -100


@contextlib.contextmanager
def parallel_state(name: Optional[str]):
    if name is None or name not in ps._STATES:
        yield
        return
    prev = ps.change_parallel_state(name)
    try:
        yield
    finally:
        ps.change_parallel_state(prev)


class _GatherVarRows(torch.autograd.Function):
    """All-gather of row blocks with different row counts per rank (backward: take own slice)."""

    @staticmethod
    def forward(ctx, x, counts, group):
        ctx.group, ctx.counts = group, counts
        r = dist.get_rank(group)
        mx = max(counts)
        pad = torch.zeros(mx, x.shape[1], dtype=x.dtype, device=x.device)
        pad[: x.shape[0]] = x
        outs = [torch.empty_like(pad) for _ in counts]
        dist.all_gather(outs, pad, group=group)
        ctx.rank = r
        return torch.cat([o[:c] for o, c in zip(outs, counts)], 0)

    @staticmethod
    def backward(ctx, g):
        start = sum(ctx.counts[: ctx.rank])
        # every rank consumed the full gathered tensor identically: sum the replicas' gradients
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[start:start + ctx.counts[ctx.rank]] / dist.get_world_size(ctx.group), None, None


class _ScaleGrad(torch.autograd.Function):
    """Identity whose backward multiplies the gradient by a constant."""

    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g * ctx.scale, None


class OmniCombinationModel(nn.Module):
    def __init__(self, lm_cfg: TransformerConfig, vit_cfg: Optional[TransformerConfig], *, image_token_id: int,
                 pre_process: bool = True, post_process: bool = True, layer_numbers=None, device=None,
                 encoder_hetero_dp: bool = False, freeze_encoder: bool = False, projector_activation: str = "gelu",
                 full_hetero_dp: bool = False,
                 vision_family: str = "qwen2_vit", vision_options: Optional[dict] = None):
        super().__init__()
        self.cfg = lm_cfg
        self.image_token_id = image_token_id
        self.pre_process, self.post_process = pre_process, post_process
        self.encoder_hetero_dp = encoder_hetero_dp
        self.foundation_model = GPTModel(lm_cfg, pre_process=pre_process, post_process=post_process,
                                         layer_numbers=layer_numbers, device=device)
        self.has_encoder = pre_process and vit_cfg is not None
        # full heterogeneous DP: EVERY rank of the model-parallel group holds the encoder (later pipeline stages as
        # replicas of the first stage's copy) and encodes its share of the step's micro-batches
        self.full_hetero_dp = full_hetero_dp and vit_cfg is not None
        if self.has_encoder or self.full_hetero_dp:
            enc_state = ENCODER_STATE if ENCODER_STATE in ps._STATES else None
            self.encoder_state = enc_state
            self.vision_family = vision_family
            with parallel_state(enc_state):
                self.encoder_model = nn.Module()
                if vision_family == "qwen2_vit":
                    self.encoder_model.image_encoder = VisionModel(vit_cfg, device=device, parallel_state=enc_state)
                    self.encoder_model.image_projector = MLPAdapter(vit_cfg, lm_cfg.hidden_size, device=device,
                                                                    activation=projector_activation)
                else:
                    # the other encoder families: one configurable ViT + the family's projector (models/vision_zoo.py)
                    from . import vision_zoo as VZ
                    opts, adapter_cls = VZ.VISION_FAMILIES[vision_family]
                    opts = {**opts, **(vision_options or {})}
                    self.encoder_model.image_encoder = VZ.GenericViT(vit_cfg, device=device, parallel_state=enc_state,
                                                                     **opts)
                    self.encoder_model.image_projector = (adapter_cls or VZ.PatchMergerAdapter)(
                        vit_cfg, lm_cfg.hidden_size, device=device)
                    n_taps = len(opts.get("deepstack_indexes", ()))
                    if n_taps:
                        self.encoder_model.deepstack_mergers = VZ.DeepStackMergers(vit_cfg, lm_cfg.hidden_size, n_taps,
                                                                                   device=device)
            if freeze_encoder:
                for p in self.encoder_model.image_encoder.parameters():
                    p.requires_grad_(False)
            if self.full_hetero_dp:
                for p in self.encoder_model.parameters():
                    # summed over the model-parallel group after the data-parallel reduction; kept in a buffer of its own
                    # so that every rank shards it identically
                    p.mp_shared = True
                    p.defer_grad_sync = True  # one encoder backward per owned micro-batch, all after the pipeline
                    if not pre_process:
                        p.shared_embedding_replica = True  # written to checkpoints and counted by the first stage only
            if encoder_hetero_dp and ps.get_state().dims.tp > 1:
                # every rank of the TP group encodes different images: its encoder gradients are partial sums, which the
                # trainer adds up over the TP group (the encoder's data-parallel degree includes the decoder's TP ranks)
                for p in self.encoder_model.parameters():
                    p.tp_partial_grad = True

    # pipeline plumbing is delegated to the language model
    @property
    def decoder(self):
        return self.foundation_model.decoder

    def set_input_tensor(self, t):
        self.foundation_model.set_input_tensor(t)

    def encode_images(self, pixels: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """[n_patches, patch_dim] -> [n_merged_tokens, lm_hidden]."""
        st = ps.get_state()
        tp, g = st.dims.tp, st.group("tp")
        n_img = grid_thw.shape[0]
        split = self.encoder_hetero_dp and tp > 1 and n_img >= tp
        if split:
            # images go to the ranks so that every rank encodes a similar number of PATCHES (longest first onto the
            # least loaded rank), not a similar number of images (reference: data/dp_balance/vit_balance.py:27-155)
            from ..data.dp_balance import balance_vit_images
            patches = (grid_thw[:, 0] * grid_thw[:, 1] * grid_thw[:, 2]).tolist()
            plan = balance_vit_images([patches] + [[] for _ in range(tp - 1)])
            by_rank = [sorted(i for (_, i) in plan[r]) for r in range(tp)]
            offs = [0]
            for n in patches:
                offs.append(offs[-1] + n)
            mine = by_rank[st.tp_rank]
            pixels = torch.cat([pixels[offs[i]:offs[i + 1]] for i in mine])
            my_grid = grid_thw[torch.tensor(mine, device=grid_thw.device)]
        else:
            my_grid = grid_thw
        self._deepstack = None
        with parallel_state(self.encoder_state):
            if self.vision_family == "qwen2_vit":
                h, widx = self.encoder_model.image_encoder(pixels, my_grid)
                emb = self.encoder_model.image_projector(h, widx)
            else:
                h, taps = self.encoder_model.image_encoder(pixels, my_grid)
                emb = self.encoder_model.image_projector(h, my_grid)
                if taps and hasattr(self.encoder_model, "deepstack_mergers"):
                    self._deepstack = self.encoder_model.deepstack_mergers(taps, my_grid)
        if self.encoder_hetero_dp and tp > 1 and not split:
            # too few images to split: every rank encoded all of them, and the gradients will still be summed over the
            # TP group, so each rank passes back 1 / tp of its (identical) gradient
            emb = _ScaleGrad.apply(emb, 1.0 / tp)
        if split:
            assert self.vision_family == "qwen2_vit", "encoder hetero-DP is implemented for the Qwen2-VL encoder"
            unit = self.encoder_model.image_projector.unit
            counts = [sum(patches[i] for i in by_rank[r]) // unit for r in range(tp)]
            emb = _GatherVarRows.apply(emb, counts, g)
            # the gathered rows are rank-major: put the images' token blocks back into image order
            toks = [p // unit for p in patches]
            pos, start = {}, 0
            for r in range(tp):
                for i in by_rank[r]:
                    pos[i] = start
                    start += toks[i]
            index = torch.cat([torch.arange(pos[i], pos[i] + toks[i], device=emb.device) for i in range(n_img)])
            emb = emb.index_select(0, index)
        return emb

    def forward(self, tokens, position_ids, *, pixels=None, grid_thw=None, labels=None, loss_mask=None, packed=None,
                loss_scale=None, image_embeds=None):
        """``image_embeds``: projected image tokens computed ahead of the pipeline (full heterogeneous DP); the encoder
        is then not run here."""
        lm = self.foundation_model
        decoder_input = None
        if self.pre_process:
            st = ps.get_state()
            sp = self.cfg.sequence_parallel and st.dims.tp > 1
            if sp:
                # full-sequence text embeddings (all-reduce), merged with the image tokens, then scattered
                emb_mod = lm.embedding.word_embeddings
                was = emb_mod.sequence_parallel
                emb_mod.sequence_parallel = False
                try:
                    x = lm.embed(tokens)
                finally:
                    emb_mod.sequence_parallel = was
            else:
                x = lm.embed(tokens)
            if image_embeds is not None:
                mask = tokens == self.image_token_id
                x = x.masked_scatter(mask.unsqueeze(-1), image_embeds.to(x.dtype))
                self.decoder.deepstack_hook = None
            elif self.has_encoder and pixels is not None and pixels.numel() > 0:
                img = self.encode_images(pixels, grid_thw).to(x.dtype)
                mask = tokens == self.image_token_id
                x = x.masked_scatter(mask.unsqueeze(-1), img)
                if getattr(self, "_deepstack", None):
                    from .vision_zoo import make_deepstack_hook
                    assert not sp, "DeepStack injection expects un-scattered hidden states"
                    self.decoder.deepstack_hook = make_deepstack_hook(self._deepstack, mask)
                else:
                    self.decoder.deepstack_hook = None
            if sp:
                x = M.scatter_to_sequence_parallel_region(x, st.group("tp"))
            decoder_input = x
        return lm(tokens, position_ids, labels=labels, loss_mask=loss_mask, packed=packed,
                  decoder_input=decoder_input, loss_scale=loss_scale)
