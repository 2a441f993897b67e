"""Supervised fine-tuning trainer for language models: chat-template datasets, sequence packing into
one packed row per micro-batch (``cu_seqlens`` + per-sequence positions), loss on assistant tokens,
optional LoRA (loongforge/train/sft/sft_llm.py:61-358, loongforge/train/sft/utils.py)."""
from __future__ import annotations

from typing import Optional

import torch

from ..data.sft import SFTDataset, sft_batch_iterator
from ..tokenizer.tokenizer import build_tokenizer
from .trainer import Trainer


def sft_paths_and_formats(args):
    """``--sft-dataset`` holds either data files (then the layout is read off the records) or, as in the reference's
    launchers, NAMES of layouts defined in ``--sft-dataset-config`` that describe the files of ``--train-data-path`` /
    ``--data-path``."""
    import os
    entries = list(args.sft_dataset)
    if all(os.path.exists(e) for e in entries):
        return entries, None
    paths = list(getattr(args, "train_data_path", None) or getattr(args, "data_path", None) or [])
    if not paths:
        raise ValueError(f"--sft-dataset {entries}: not files, and no --data-path / --train-data-path names the files they describe")
    from ..data.sft_formats import resolve_formats
    names = list(getattr(args, "sft_train_dataset", None) or entries)
    return paths, resolve_formats(names, len(paths), getattr(args, "sft_dataset_config", None))


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
        paths, formats = sft_paths_and_formats(args)
        if getattr(args, "sft_data_streaming", False):
            from ..data.sft import streaming_sft_batch_iterator
            return streaming_sft_batch_iterator(
                paths, tok, self.tcfg.seq_length, template=args.chat_template or "chatml",
                buffer_size=int(getattr(args, "streaming_buffer_size", 16384) or 16384),
                strategy=getattr(args, "sft_data_mix_strategy", "concat") or "concat", formats=formats,
                train_on_prompt=args.train_on_prompt, packing=args.packing_sft_data, dp_rank=self.st.dp_rank,
                dp_size=self.st.dp_size, seed=self.tcfg.seed, pad_id=tok.pad,
                start_sample=self.consumed_samples // max(self.st.dp_size, 1))
        ds = SFTDataset(paths, tok, template=args.chat_template or "chatml", max_len=self.tcfg.seq_length,
                        train_on_prompt=args.train_on_prompt, seed=self.tcfg.seed, formats=formats)
        vpaths = list(getattr(args, "valid_data_path", None) or [])
        if vpaths and self.tcfg.eval_interval and self.tcfg.eval_iters:
            vformats = None
            if formats is not None:
                from ..data.sft_formats import resolve_formats
                vformats = resolve_formats(list(getattr(args, "sft_valid_dataset", None) or [f.name for f in formats][:1]),
                                           len(vpaths), getattr(args, "sft_dataset_config", None))
            vds = SFTDataset(vpaths, tok, template=args.chat_template or "chatml", max_len=self.tcfg.seq_length,
                             train_on_prompt=args.train_on_prompt, seed=self.tcfg.seed, formats=vformats)
            self.valid_iterator = sft_batch_iterator(vds, self.tcfg.seq_length, packing=args.packing_sft_data, dp_rank=self.st.dp_rank,
                                                     dp_size=self.st.dp_size, seed=self.tcfg.seed + 1, pad_id=tok.pad, pad_to_multiple=1)
        return sft_batch_iterator(ds, self.tcfg.seq_length, packing=args.packing_sft_data, dp_rank=self.st.dp_rank,
                                  dp_size=self.st.dp_size, seed=self.tcfg.seed, pad_id=tok.pad,
                                  start_sample=self.consumed_samples // max(self.st.dp_size, 1),
                                  pad_to_multiple=1,  # rows are padded to seq_length, which the parallel sizes divide
                                  balance_group=(self.tcfg.global_batch_size
                                                 if (getattr(args, "group_by_length", False)
                                                     or getattr(args, "sft_sort_batch", False)) else 0))
