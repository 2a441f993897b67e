"""Megatron ``.bin`` / ``.idx`` indexed token datasets (writer, memory-mapped reader) and the GPT
sample index that cuts the concatenated token stream into ``seq_length + 1`` windows
(what tools/data_preprocess/llm/preprocess_pretrain_data.py produces and ``GPTDataset`` consumes,
loongforge/train/pretrain/pretrain_llm.py:183-233)."""
from __future__ import annotations

import os
import struct
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


class IndexedDatasetWriter:
    def __init__(self, prefix: str, dtype=np.int32):
        self.prefix, self.dtype = prefix, np.dtype(dtype)
        self._bin = open(prefix + ".bin", "wb")
        self.sizes: List[int] = []
        self.doc_idx: List[int] = [0]

    def add_document(self, tokens: Sequence[int]):
        arr = np.asarray(tokens, dtype=self.dtype)
        self._bin.write(arr.tobytes(order="C"))
        self.sizes.append(len(arr))
        self.doc_idx.append(len(self.sizes))

    def add_sentences(self, sentences: Sequence[Sequence[int]]):
        """One document made of several sequences (sentence-split corpora): every sentence is an item of its own, the
        document index marks where the document ends."""
        for sent in sentences:
            arr = np.asarray(sent, dtype=self.dtype)
            self._bin.write(arr.tobytes(order="C"))
            self.sizes.append(len(arr))
        self.doc_idx.append(len(self.sizes))

    def merge(self, prefix: str):
        """Appends another data set of the same dtype (partition files of a parallel pre-processing run)."""
        other = IndexedDataset(prefix)
        assert other.dtype == self.dtype, f"{prefix}: dtype {other.dtype} != {self.dtype}"
        base = len(self.sizes)
        with open(prefix + ".bin", "rb") as f:
            while True:
                chunk = f.read(1 << 24)
                if not chunk:
                    break
                self._bin.write(chunk)
        self.sizes.extend(int(x) for x in other.sizes)
        self.doc_idx.extend(int(d) + base for d in other.doc_idx[1:])

    def finalize(self):
        self._bin.close()
        with open(self.prefix + ".idx", "wb") as f:
            f.write(_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", _CODES[self.dtype]))
            f.write(struct.pack("<Q", len(self.sizes)))
            f.write(struct.pack("<Q", len(self.doc_idx)))
            sizes = np.asarray(self.sizes, dtype=np.int32)
            f.write(sizes.tobytes(order="C"))
            pointers = np.zeros(len(sizes), dtype=np.int64)
            if len(sizes) > 1:
                np.cumsum(sizes[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self.doc_idx, dtype=np.int64).tobytes(order="C"))


class IndexedDataset:
    def __init__(self, prefix: str):
        with open(prefix + ".idx", "rb") as f:
            assert f.read(9) == _MAGIC, "not a Megatron index file"
            (version,) = struct.unpack("<Q", f.read(8))
            (code,) = struct.unpack("<B", f.read(1))
            (n,) = struct.unpack("<Q", f.read(8))
            (ndoc,) = struct.unpack("<Q", f.read(8))
            off = f.tell()
        self.dtype = np.dtype(_DTYPES[code])
        idx = np.memmap(prefix + ".idx", mode="r", order="C")
        self.sizes = np.frombuffer(idx, dtype=np.int32, count=n, offset=off)
        self.pointers = np.frombuffer(idx, dtype=np.int64, count=n, offset=off + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(idx, dtype=np.int64, count=ndoc, offset=off + self.sizes.nbytes + self.pointers.nbytes)
        self.data = np.memmap(prefix + ".bin", mode="r", order="C", dtype=self.dtype)

    def __len__(self):
        return len(self.sizes)

    def __getitem__(self, i) -> np.ndarray:
        start = self.pointers[i] // self.dtype.itemsize
        return self.data[start:start + self.sizes[i]]

    @property
    def num_tokens(self) -> int:
        return int(self.sizes.astype(np.int64).sum())


class GPTDataset:
    """Samples of seq_length+1 tokens from the shuffled document stream (documents concatenated
    with an end-of-document token already inside them)."""

    def __init__(self, indexed: IndexedDataset, seq_length: int, num_samples: int, seed: int = 1234,
                 eod_token: Optional[int] = None, eod_mask_loss: bool = False,
                 doc_range: Optional[Tuple[int, int]] = None):
        """``doc_range``: half-open range of document indices this split may draw from (train / valid / test)."""
        self.ds, self.seq_length, self.eod, self.eod_mask_loss = indexed, seq_length, eod_token, eod_mask_loss
        rng = np.random.RandomState(seed)
        lo, hi = doc_range if doc_range is not None else (0, len(indexed))
        if hi <= lo:
            raise ValueError(f"empty document range {doc_range} for a dataset of {len(indexed)} documents")
        tokens_per_epoch = int(sum(len(indexed[d]) for d in range(lo, hi)))
        epochs = max(1, -(-(num_samples * seq_length + 1) // max(tokens_per_epoch, 1)))
        docs = np.concatenate([lo + rng.permutation(hi - lo) for _ in range(epochs)])
        self.stream = np.concatenate([np.asarray(indexed[d]) for d in docs]).astype(np.int64)
        self.num_samples = min(num_samples, (len(self.stream) - 1) // seq_length)
        self.shuffle = rng.permutation(self.num_samples)

    def __len__(self):
        return self.num_samples

    def __getitem__(self, i) -> Dict[str, torch.Tensor]:
        j = int(self.shuffle[i % self.num_samples])
        w = torch.from_numpy(self.stream[j * self.seq_length:(j + 1) * self.seq_length + 1].copy())
        tokens, labels = w[:-1], w[1:]
        mask = torch.ones(self.seq_length)
        if self.eod_mask_loss and self.eod is not None:
            mask[tokens == self.eod] = 0.0
        return {"tokens": tokens, "labels": labels, "loss_mask": mask,
                "position_ids": torch.arange(self.seq_length)}


def gpt_batch_iterator(ds: GPTDataset, micro_batch_size: int, *, dp_rank=0, dp_size=1, start_sample=0,
                       pin_memory=False) -> Iterator[Dict[str, torch.Tensor]]:
    step = 0
    while True:
        base = start_sample + (step * dp_size + dp_rank) * micro_batch_size
        items = [ds[base + j] for j in range(micro_batch_size)]
        batch = {k: torch.stack([it[k] for it in items]) for k in items[0]}
        if pin_memory:
            batch = {k: v.pin_memory() for k, v in batch.items()}
        batch["num_valid_tokens"] = int(batch["loss_mask"].sum().item())
        yield batch
        step += 1


def split_document_ranges(num_docs: int, split: str) -> List[Tuple[int, int]]:
    """``"949,50,1"`` -> [(0, a), (a, b), (b, num_docs)]: train / validation / test document ranges in the ratio
    given (Megatron's ``--split``)."""
    w = [float(x) for x in split.replace("/", ",").split(",") if x.strip() != ""]
    w = (w + [0.0, 0.0, 0.0])[:3]
    tot = sum(w)
    if tot <= 0:
        raise ValueError(f"bad split {split!r}")
    bounds, acc = [0], 0.0
    for x in w:
        acc += x / tot
        bounds.append(int(round(acc * num_docs)))
    bounds[-1] = num_docs
    return [(bounds[i], max(bounds[i], bounds[i + 1])) for i in range(3)]


class BlendedDataset:
    """Weighted mixture of datasets: sample i comes from the dataset whose share of the first i samples lags its
    weight the most (the deterministic scheme of Megatron's blending indices), so every prefix of the stream has
    the requested proportions."""

    def __init__(self, datasets: Sequence, weights: Sequence[float], num_samples: int):
        assert len(datasets) == len(weights) and datasets
        w = np.asarray(weights, dtype=np.float64)
        w = w / w.sum()
        self.datasets = list(datasets)
        counts = np.zeros(len(w), dtype=np.int64)
        self.which = np.empty(num_samples, dtype=np.int32)
        self.index = np.empty(num_samples, dtype=np.int64)
        for i in range(num_samples):
            d = int(np.argmax(w * (i + 1) - counts))
            self.which[i], self.index[i] = d, counts[d]
            counts[d] += 1

    def __len__(self):
        return len(self.which)

    def __getitem__(self, i):
        i = i % len(self.which)
        return self.datasets[int(self.which[i])][int(self.index[i])]


def parse_data_path(data_path: Sequence[str]) -> Tuple[List[float], List[str]]:
    """``["a"]`` -> ([1.0], ["a"]); ``["0.3", "a", "0.7", "b"]`` -> ([0.3, 0.7], ["a", "b"])."""
    items = list(data_path)
    if len(items) == 1:
        return [1.0], items
    if len(items) % 2:
        raise ValueError("--data-path takes one prefix, or weight / prefix pairs")
    return [float(x) for x in items[0::2]], list(items[1::2])


def build_gpt_datasets(data_path: Sequence[str], split: str, seq_length: int, samples: Sequence[int], seed: int = 1234,
                       eod_token: Optional[int] = None, eod_mask_loss: bool = False):
    """(train, valid, test) datasets over one or several ``.bin/.idx`` prefixes; a split with no documents or no
    requested samples is None (reference: Megatron ``BlendedMegatronDatasetBuilder`` as used by
    loongforge/train/pretrain/pretrain_llm.py:198-229)."""
    weights, prefixes = parse_data_path(data_path)
    indexed = [IndexedDataset(p) for p in prefixes]
    out = []
    for si in range(3):
        n = int(samples[si])
        parts, ws = [], []
        for w, ds in zip(weights, indexed):
            lo, hi = split_document_ranges(len(ds), split)[si]
            if hi > lo and n > 0:
                share = max(1, int(np.ceil(n * w / sum(weights) * 1.005)) + 1)
                parts.append(GPTDataset(ds, seq_length, share, seed + si, eod_token, eod_mask_loss, (lo, hi)))
                ws.append(w)
        if not parts:
            out.append(None)
        elif len(parts) == 1:
            out.append(parts[0])
        else:
            out.append(BlendedDataset(parts, ws, n))
    return tuple(out)
