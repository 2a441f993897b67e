"""Supervised fine-tuning trainer for language models: chat-template datasets, sequence packing into
one packed row per micro-batch (``cu_seqlens`` + per-sequence positions), loss on assistant tokens,
optional LoRA (loongforge/train/sft/sft_llm.py:61-358, loongforge/train/sft/utils.py)."""
from __future__ import annotations

from typing import Optional

import torch

from ..data.sft import SFTDataset, sft_batch_iterator
from ..tokenizer.tokenizer import build_tokenizer
from .trainer import Trainer


class SFTTrainer(Trainer):
    def __init__(self, model_cfg, train_cfg, dims=None, *, lora: Optional[dict] = None, **kw):
        self._lora = lora
        super().__init__(model_cfg, train_cfg, dims, **kw)

    def _default_model_provider(self, pre_process, post_process, layer_numbers):
        model = super()._default_model_provider(pre_process, post_process, layer_numbers)
        if self._lora:
            from ..models.peft import apply_lora
            apply_lora(model, **self._lora)
        return model

    def build_data_iterator(self, args):
        if getattr(args, "mock_data", False) or not getattr(args, "sft_dataset", None):
            return None
        tok = build_tokenizer(args.tokenizer_type, args.hf_tokenizer_path, use_fast=args.use_fast_tokenizer)
        ds = SFTDataset(args.sft_dataset, tok, template=args.chat_template or "chatml", max_len=self.tcfg.seq_length,
                        train_on_prompt=args.train_on_prompt, seed=self.tcfg.seed)
        return sft_batch_iterator(ds, self.tcfg.seq_length, packing=args.packing_sft_data, dp_rank=self.st.dp_rank,
                                  dp_size=self.st.dp_size, seed=self.tcfg.seed, pad_id=tok.pad,
                                  start_sample=self.consumed_samples // max(self.st.dp_size, 1),
                                  pad_to_multiple=1,  # rows are padded to seq_length, which the parallel sizes divide
                                  balance_group=(self.tcfg.global_batch_size
                                                 if (getattr(args, "group_by_length", False)
                                                     or getattr(args, "sft_sort_batch", False)) else 0))
