"""Supervised fine-tuning datasets: jsonl/json files in alpaca / sharegpt / openai formats, blended
by weight, tokenised with a chat template, optionally packed
(loongforge/data/sft_dataset.py, sft_data_collator.py, blended_hf_dataset_builder.py)."""
from __future__ import annotations

import json
import random
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

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


# ---------------------------------------------------------------------------------------------- streaming
def _stream_records(path: str) -> Iterator[dict]:
    """JSONL records of one file, one at a time (a JSON array is read whole: it cannot be streamed)."""
    with open(path) as f:
        head = f.read(1)
        f.seek(0)
        if head == "[":
            yield from json.load(f)
            return
        for line in f:
            if line.strip():
                yield json.loads(line)


def mixed_record_stream(paths: Sequence[str], strategy: str = "concat", formats: Optional[Sequence] = None) -> Iterator[dict]:
    """One pass over several files: ``concat`` reads them one after another; ``interleave_under`` takes one record of each
    in turn and stops when the SHORTEST file ends; ``interleave_over`` goes on until the LONGEST one ends, restarting the
    shorter files (reference: --sft-data-mix-strategy, loongforge/data/blended_hf_dataset_builder.py:240-265)."""
    def tagged(i):
        for r in _stream_records(paths[i]):
            yield dict(r, __format__=formats[i]) if formats is not None else r

    if strategy == "concat" or len(paths) == 1:
        for i in range(len(paths)):
            yield from tagged(i)
        return
    if strategy not in ("interleave_under", "interleave_over"):
        raise ValueError(f"unknown mix strategy {strategy!r}")
    its = [tagged(i) for i in range(len(paths))]
    finished = [False] * len(paths)
    while True:
        for i in range(len(its)):
            try:
                rec = next(its[i])
            except StopIteration:
                finished[i] = True
                if strategy == "interleave_under" or all(finished):
                    return
                its[i] = tagged(i)
                rec = next(its[i], None)
                if rec is None:
                    continue
            yield rec


def streaming_sft_batch_iterator(paths: Sequence[str], tokenizer, seq_length: int, *, template: str = "chatml",
                                 buffer_size: int = 16384, strategy: str = "concat", formats: Optional[Sequence] = None,
                                 train_on_prompt: bool = False, packing: bool = True, dp_rank: int = 0, dp_size: int = 1,
                                 seed: int = 1234, pad_id: int = 0, pad_to_multiple: int = 1,
                                 start_sample: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """SFT micro-batches without loading the data set: records stream through a shuffle buffer of ``buffer_size`` (a
    random slot is emitted and refilled), record k goes to rank ``k % dp_size``, tokenised samples are packed greedily
    into rows of ``seq_length`` as they arrive. Passes over the data repeat for ever with another shuffle seed
    (``--sft-data-streaming``, ``--streaming-buffer-size``)."""
    helper = SFTDataset.__new__(SFTDataset)
    helper.tokenizer, helper.template, helper.max_len = tokenizer, template, seq_length
    helper.train_on_prompt, helper.fmt = train_on_prompt, "auto"
    skip, epoch = start_sample, 0
    while True:
        rng = random.Random(seed + epoch)
        buf: List[dict] = []
        row: List[Tuple[List[int], List[int]]] = []
        used = 0

        def emit(rec, k):
            nonlocal row, used, skip
            if k % dp_size != dp_rank:
                return None
            helper.records = [rec]
            ids, labels = helper[0]
            ids, labels = ids[:seq_length], labels[:seq_length]
            out = None
            if not packing:
                out = [(ids, labels)]
            elif used + len(ids) > seq_length and row:
                out, row, used = row, [], 0
            if packing:
                row.append((ids, labels))
                used += len(ids)
            return out

        k = 0
        for rec in mixed_record_stream(paths, strategy, formats):
            if len(buf) < buffer_size:
                buf.append(rec)
                continue
            j = rng.randrange(len(buf))
            ready = emit(buf[j], k)
            buf[j] = rec
            k += 1
            if ready:
                if skip > 0:
                    skip -= 1
                else:
                    yield collate_packed(ready, seq_length, pad_id, pad_to_multiple)
        rng.shuffle(buf)
        for rec in buf:
            ready = emit(rec, k)
            k += 1
            if ready:
                if skip > 0:
                    skip -= 1
                else:
                    yield collate_packed(ready, seq_length, pad_id, pad_to_multiple)
        if row:
            if skip > 0:
                skip -= 1
            else:
                yield collate_packed(row, seq_length, pad_id, pad_to_multiple)
        if k == 0:
            raise ValueError(f"no records in {list(paths)}")
        epoch += 1
