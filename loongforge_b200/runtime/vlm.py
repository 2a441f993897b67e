"""Vision-language trainer (pre-training and SFT): builds the ViT + projector + LLM composition with
a separate parallel state for the encoder, feeds packed text + image batches, computes the loss on
text positions only (loongforge/train/pretrain/pretrain_vlm.py:78-521, loongforge/train/sft/sft_vlm.py)."""
from __future__ import annotations

from typing import Dict, Iterator, Optional

import torch
import torch.distributed as dist

from ..data.position_ids import mrope_ids
from ..models.config import TransformerConfig
from ..models.omni import ENCODER_STATE, OmniCombinationModel
from ..models.registry import get_model_config
from ..models.transformer import PackedSeqParams
from ..parallel import state as ps
from ..parallel.state import ParallelDims
from .trainer import Trainer


def synthetic_vlm_iterator(vocab_size: int, seq_length: int, *, images_per_sample: int = 4, image_size: int = 448,
                           patch: int = 14, temporal_patch: int = 2, merge: int = 2, channels: int = 3,
                           image_token_id: Optional[int] = None, dp_rank: int = 0, dp_size: int = 1, seed: int = 1234,
                           pin_memory: Optional[bool] = None) -> Iterator[Dict[str, torch.Tensor]]:
    """Packed samples: `images_per_sample` synthetic images (pixels ~ N(0,1), already patchified to
    ``[n_patches, C*t*p*p]``) whose merged tokens are interleaved with uniform random text tokens up
    to `seq_length`; labels are -100 (masked) on image positions."""
    image_token_id = vocab_size - 1 if image_token_id is None else image_token_id
    g = image_size // patch
    tokens_per_image = (g // merge) ** 2
    n_patch = g * g
    pin = torch.cuda.is_available() if pin_memory is None else pin_memory
    step = 0
    text_total = seq_length - images_per_sample * tokens_per_image
    assert text_total > images_per_sample, "sequence too short for the images"
    while True:
        gen = torch.Generator()
        gen.manual_seed(seed * 7919 + step * dp_size + dp_rank)
        toks = torch.randint(0, vocab_size - 1, (seq_length + 1,), generator=gen)
        seg = text_total // (images_per_sample + 1)
        pos = 0
        tokens = toks[:-1].clone()
        for i in range(images_per_sample):
            pos += seg
            tokens[pos:pos + tokens_per_image] = image_token_id
            pos += tokens_per_image
        labels = toks[1:].clone()
        # no loss where the INPUT or the TARGET is an image placeholder
        is_img = tokens == image_token_id
        nxt_img = torch.cat([is_img[1:], is_img.new_zeros(1)])
        mask = (~is_img & ~nxt_img).float()
        pixels = torch.randn(images_per_sample * n_patch, channels * temporal_patch * patch * patch, generator=gen)
        grid = torch.tensor([[1, g, g]] * images_per_sample)
        batch = {"tokens": tokens.unsqueeze(0), "labels": labels.unsqueeze(0), "loss_mask": mask.unsqueeze(0),
                 "position_ids": mrope_ids(tokens, grid, image_token_id, merge).unsqueeze(1),  # [3, 1, T]
                 "pixels": pixels, "grid_thw": grid}
        if pin:
            batch = {k: v.pin_memory() for k, v in batch.items()}
        batch["num_valid_tokens"] = int(mask.sum().item())
        yield batch
        step += 1


class VLMTrainer(Trainer):
    def __init__(self, model_cfg: TransformerConfig, train_cfg, dims: Optional[ParallelDims] = None, *,
                 vit_cfg: Optional[TransformerConfig] = None, encoder_tp: int = 1, encoder_hetero_dp: bool = False,
                 image_token_id: Optional[int] = None, encoder_recompute: bool = True,
                 vision_family: str = "qwen2_vit", vision_options: Optional[dict] = None, freeze_encoder: bool = False,
                 images_per_sample: int = 4, image_size: int = 448, full_hetero_dp: bool = False,
                 full_hetero_cpu_offload: bool = False, lora: Optional[dict] = None, **kw):
        """``vision_family``: ``qwen2_vit`` (Qwen2/2.5-VL encoder) or a key of ``models.vision_zoo.VISION_FAMILIES``
        (Qwen3-VL, InternViT, RICE, Moon, ERNIE, MiniCPM-V encoders with their projectors)."""
        self.vit_cfg = vit_cfg or get_model_config("qwen2.5-vit")
        self.vision_family, self.vision_options, self.freeze_encoder = vision_family, vision_options, freeze_encoder
        self.images_per_sample, self.image_size = images_per_sample, image_size
        if encoder_recompute:
            self.vit_cfg.recompute_granularity = "full"
        self.encoder_hetero_dp = encoder_hetero_dp
        self._lora = lora  # adapters on the language model's linears; its base weights are frozen
        self.full_hetero_dp, self.full_hetero_cpu_offload = full_hetero_dp, full_hetero_cpu_offload
        if full_hetero_dp and ((dims and dims.cp > 1) or encoder_tp != 1 or encoder_hetero_dp):
            raise ValueError("full heterogeneous DP needs cp = 1 and encoder TP 1, and replaces encoder hetero-DP")
        self.image_token_id = model_cfg.vocab_size - 1 if image_token_id is None else image_token_id
        dims = dims or ParallelDims()
        if not ps.model_parallel_is_initialized():
            ps.initialize_model_parallel(dims)
            from ..parallel.context_parallel import ensure_cp_groups
            ensure_cp_groups()
            # the encoder gets its own tensor-parallel degree (must divide the decoder's)
            ps.create_parallel_state(ENCODER_STATE, ParallelDims(tp=encoder_tp, pp=dims.pp, cp=dims.cp))
        if train_cfg.bf16:
            self.vit_cfg.params_dtype = torch.bfloat16
        super().__init__(model_cfg, train_cfg, dims, **kw)
        self._mp_shared = [p for m in self.models for p in m.module.parameters() if getattr(p, "mp_shared", False)]
        if self._mp_shared and self.st.group("mp") is not None:
            self.optimizer.post_sync_hooks.append(self._allreduce_mp_shared_grads)

    def _allreduce_mp_shared_grads(self):
        """Full hetero-DP: every rank of the model-parallel group back-propagated the encoder for ITS micro-batches;
        the sum over the group is the gradient of the step."""
        g = self.st.group("mp")
        for p in self._mp_shared:
            dist.all_reduce(p.main_grad, group=g)

    def _default_model_provider(self, pre_process, post_process, layer_numbers):
        model = self._build_omni(pre_process, post_process, layer_numbers)
        if self._lora:
            # adapters per component: {"apply_to_image_encoder": True, ...} next to the usual rank / alpha / targets
            from ..models.peft import apply_vlm_lora
            done = apply_vlm_lora(model, frozen=("image_encoder",) if self.freeze_encoder else (), **self._lora)
            if self.st.rank == 0:
                n_train = sum(p.numel() for p in model.parameters() if p.requires_grad)
                print(" > LoRA adapters: " + ", ".join(f"{k}: {len(v)} linears" for k, v in done.items())
                      + f"; {n_train:,d} trainable parameters of {sum(p.numel() for p in model.parameters()):,d}", flush=True)
        return model

    def _build_omni(self, pre_process, post_process, layer_numbers):
        return OmniCombinationModel(self.mcfg, self.vit_cfg if (pre_process or self.full_hetero_dp) else None,
                                    full_hetero_dp=self.full_hetero_dp, image_token_id=self.image_token_id,
                                    pre_process=pre_process, post_process=post_process, layer_numbers=layer_numbers,
                                    device=self.device, encoder_hetero_dp=self.encoder_hetero_dp,
                                    vision_family=self.vision_family, vision_options=self.vision_options,
                                    freeze_encoder=self.freeze_encoder)

    def build_data_iterator(self, args=None):
        st = self.st
        v = self.vit_cfg
        paths = getattr(args, "data_path", None) if args is not None else None
        if paths:
            # image-text shards (tools/data_preprocess/vlm_to_webdataset.py) -> task encoder -> online packer
            from ..data.multimodal import VLMTaskEncoder, VisionPreprocess, vlm_batch_iterator, webdataset_samples
            from ..tokenizer.tokenizer import build_tokenizer
            tok = build_tokenizer(args.tokenizer_type, args.hf_tokenizer_path, use_fast=args.use_fast_tokenizer)
            vision = VisionPreprocess(patch_size=v.patch_size, temporal_patch_size=v.temporal_patch_size,
                                      merge_size=v.spatial_merge_size,
                                      **{k: getattr(args, k) for k in ("min_pixels", "max_pixels")
                                         if getattr(args, k, None) is not None})
            # the family of the vision tower decides how an image becomes tokens (data/task_encoders.py)
            from ..data.task_encoders import TASK_ENCODERS, SpecialTokens, build_task_encoder
            if self.vision_family in TASK_ENCODERS:
                def special(name):
                    try:
                        ids = tok.tokenize(name)
                    except Exception:  # noqa: BLE001
                        return None
                    return ids[0] if len(ids) == 1 else None
                enc = build_task_encoder(self.vision_family, lambda text: tok.tokenize(text),
                                         SpecialTokens(image=self.image_token_id, video=special("<|video_pad|>"),
                                                       vision_start=special("<|vision_start|>"),
                                                       vision_end=special("<|vision_end|>"), eos=tok.eod),
                                         vision, max_length=self.tcfg.seq_length)
            else:
                enc = VLMTaskEncoder(lambda text: tok.tokenize(text), self.image_token_id, vision, eos_id=tok.eod)
            samples = webdataset_samples(paths[-1], dp_rank=st.dp_rank, dp_size=st.dp_size, seed=self.tcfg.seed,
                                         start_sample=self.consumed_samples // max(st.dp_size, 1),
                                         frame_num=getattr(args, "frame_num", None), fps=getattr(args, "fps", None))
            return vlm_batch_iterator(samples, enc, self.tcfg.seq_length, merge_size=v.spatial_merge_size,
                                      pad_id=tok.pad, packing=bool(getattr(args, "packing_sft_data", True)),
                                      buffer_size=int(getattr(args, "packing_batch_size", None) or 16),
                                      pin_memory=self.device.type == "cuda")
        return synthetic_vlm_iterator(self.mcfg.vocab_size, self.tcfg.seq_length, patch=v.patch_size,
                                      temporal_patch=v.temporal_patch_size, merge=v.spatial_merge_size,
                                      channels=v.in_channels, image_token_id=self.image_token_id, dp_rank=st.dp_rank,
                                      dp_size=st.dp_size, seed=self.tcfg.seed, images_per_sample=self.images_per_sample,
                                      image_size=self.image_size)

    def _default_forward_step(self, data_iterator, model):
        b = self.get_batch(data_iterator)
        tokens = b["tokens"].reshape(-1)
        labels = b["labels"].reshape(-1)
        mask = b["loss_mask"].reshape(-1)
        pos = b["position_ids"].reshape(3, -1)
        nmb = self.mb_calc.num_microbatches
        n_valid = max(int(b.get("num_valid_tokens", mask.numel())), 1)
        scale = 1.0 / (n_valid * nmb)
        packed = PackedSeqParams(cu_seqlens=b["cu_seqlens"]) if "cu_seqlens" in b else None
        first = self.st.is_first_stage
        embeds = b.get("image_embeds")
        out = model(tokens, pos, pixels=b["pixels"].to(self.mcfg.params_dtype) if (first and embeds is None) else None,
                    grid_thw=b["grid_thw"] if first else None, labels=labels, loss_mask=mask, packed=packed,
                    loss_scale=scale, **({"image_embeds": embeds} if (first and embeds is not None) else {}))

        def loss_func(losses):
            loss = (losses * mask.float()).sum() * scale
            return loss, {"lm loss": loss.detach() * nmb, "num_tokens": n_valid}

        return out, loss_func

    # ------------------------------------------------------------------ full heterogeneous DP
    def train_step(self, data_iterator):
        if not self.full_hetero_dp:
            return super().train_step(data_iterator)
        return self._train_step_full_hetero(data_iterator)

    def _train_step_full_hetero(self, data_iterator):
        """All encoder rounds run BEFORE the pipeline: the ranks of the model-parallel group (TP x PP, which all see the
        same micro-batches) each encode the micro-batches they own and broadcast the embeddings; the pipeline then runs
        on precomputed embeddings; afterwards the embedding gradients return to their owners, which run the encoder
        backward. The encoder's gradients are summed over the model-parallel group in the optimizer's post-sync hook
        (reference: loongforge/train/training_utils.py:1484-1677,1720-1841)."""
        from .hetero_dp import FullHeteroEncoderRunner

        st = self.st
        nmb = self.mb_calc.num_microbatches
        if self.tcfg.dp_balance and st.dp_size > 1:
            data_iterator = self._balanced(data_iterator)
        batches = [self.get_batch(data_iterator) for _ in range(nmb)]
        module = self.models[0].module
        dt = self.mcfg.params_dtype

        def encode(inp):
            pixels, grid = inp
            return module.encode_images(pixels.to(dt), grid)

        offloader = None
        if self.full_hetero_cpu_offload:
            from .offload import AsyncCPUOffloader
            offloader = AsyncCPUOffloader()
        runner = FullHeteroEncoderRunner(st.group("mp"), encode, offloader=offloader)
        runner.encode_all([(b["pixels"], b["grid_thw"]) for b in batches])

        def feed():
            for i, b in enumerate(batches):
                b["image_embeds"] = runner.leaf(i)  # reloaded from host memory here when offloading
                yield b

        self._hetero_runner, self._already_balanced = runner, True
        try:
            return super().train_step(feed())
        finally:
            self._hetero_runner, self._already_balanced = None, False

    def _before_optimizer_step(self):
        # runs right after the pipeline's backward and before the optimizer: the point where the embedding gradients go
        # back to the ranks that encoded them (the first stage's first TP rank holds the complete gradient)
        runner = getattr(self, "_hetero_runner", None)
        if runner is not None:
            runner.backward(contributes=self.st.is_first_stage and self.st.tp_rank == 0)
