"""Supervised fine-tuning datasets: jsonl/json files in alpaca / sharegpt / openai formats, blended
by weight, tokenised with a chat template, optionally packed
(loongforge/data/sft_dataset.py, sft_data_collator.py, blended_hf_dataset_builder.py)."""
from __future__ import annotations

import json
import random
from typing import Dict, Iterator, List, Optional, Sequence

import torch

from .chat_template import encode_chat, to_messages
from .packing import collate_packed, pack_first_fit_decreasing


def load_records(path: str) -> List[dict]:
    with open(path) as f:
        head = f.read(1)
        f.seek(0)
        if head == "[":
            return json.load(f)
        return [json.loads(line) for line in f if line.strip()]


class SFTDataset:
    def __init__(self, paths: Sequence[str], tokenizer, template: str = "chatml", max_len: int = 2048,
                 weights: Optional[Sequence[float]] = None, fmt: str = "auto", train_on_prompt: bool = False,
                 seed: int = 1234, formats: Optional[Sequence] = None):
        """``formats``: one ``sft_formats.DatasetFormat`` per path (named layouts of ``--sft-dataset``); without it the
        layout is guessed from the record's keys (``fmt``)."""
        self.tokenizer, self.template, self.max_len = tokenizer, template, max_len
        self.train_on_prompt, self.fmt = train_on_prompt, fmt
        sets = [load_records(p) for p in paths]
        if formats is not None:
            assert len(formats) == len(sets)
            sets = [[dict(r, __format__=f) for r in s] for s, f in zip(sets, formats)]
        if weights is None:
            self.records = [r for s in sets for r in s]
        else:  # blend: sample each source proportionally to its weight
            rng = random.Random(seed)
            total = sum(len(s) for s in sets)
            wsum = float(sum(weights))
            self.records = []
            for s, w in zip(sets, weights):
                n = max(1, round(total * w / wsum))
                self.records.extend(rng.choices(s, k=n) if n > len(s) else rng.sample(s, n))
            rng.shuffle(self.records)

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        rec = self.records[i]
        if "input_ids" in rec:  # tokenised offline (tools/data_preprocess/preprocess_sft_data.py): used as it is
            ids, labels = list(rec["input_ids"]), list(rec.get("labels") or rec["input_ids"])
            return ids[:self.max_len], labels[:self.max_len]
        if "__format__" in rec:
            from .sft_formats import convert
            msgs, tools, _ = convert(rec, rec["__format__"])
            return encode_chat(self.tokenizer, msgs, self.template, self.train_on_prompt, self.max_len, tools=tools)
        return encode_chat(self.tokenizer, to_messages(rec, self.fmt), self.template, self.train_on_prompt,
                           self.max_len, tools=rec.get("tools"))


def sft_batch_iterator(ds: SFTDataset, seq_length: int, *, packing: bool = True, dp_rank: int = 0, dp_size: int = 1,
                       seed: int = 1234, pad_id: int = 0, start_sample: int = 0,
                       pad_to_multiple: int = 1, balance_group: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Infinite iterator of micro-batches of ONE packed row of `seq_length` tokens (or one padded
    sample when packing is off). Epochs are reshuffled deterministically; rank r takes every
    dp_size-th bin. With ``balance_group`` = G > 0 (``--group-by-length`` / ``--sft-sort-batch``) every G consecutive
    samples of the shuffled order are split over the data-parallel ranks by cost (length squared) before packing, so
    that ranks finish their share of a step together (data/samplers.py::BalancedGroupSampler)."""
    epoch, consumed = 0, start_sample
    if balance_group > 0:
        from .samplers import BalancedGroupSampler
        samples = [ds[i] for i in range(len(ds))]
        sampler = BalancedGroupSampler([len(s[0]) for s in samples], min(balance_group, len(samples)), dp_size, dp_rank,
                                       seq_length, seed=seed)
        for packs in sampler:
            for pack in packs:
                if consumed > 0:
                    consumed -= 1
                    continue
                yield collate_packed([(samples[i][0][:seq_length], samples[i][1][:seq_length]) for i in pack],
                                     seq_length, pad_id, pad_to_multiple)
    while True:
        rng = random.Random(seed + epoch)
        order = list(range(len(ds)))
        rng.shuffle(order)
        samples = [ds[i] for i in order]
        if packing:
            bins = pack_first_fit_decreasing([len(s[0]) for s in samples], seq_length)
        else:
            bins = [[i] for i in range(len(samples))]
        for b in range(dp_rank, len(bins) - (len(bins) % dp_size if len(bins) >= dp_size else 0), dp_size):
            if consumed > 0:
                consumed -= 1
                continue
            yield collate_packed([samples[i] for i in bins[b]], seq_length, pad_id, pad_to_multiple)
        epoch += 1
