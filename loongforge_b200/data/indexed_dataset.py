"""Megatron ``.bin`` / ``.idx`` indexed token datasets (writer, memory-mapped reader) and the GPT
sample index that cuts the concatenated token stream into ``seq_length + 1`` windows
(what tools/data_preprocess/llm/preprocess_pretrain_data.py produces and ``GPTDataset`` consumes,
loongforge/train/pretrain/pretrain_llm.py:183-233)."""
from __future__ import annotations

import os
import struct
from typing import Dict, Iterator, List, Optional, Sequence

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
                 eod_token: Optional[int] = None, eod_mask_loss: bool = False):
        self.ds, self.seq_length, self.eod, self.eod_mask_loss = indexed, seq_length, eod_token, eod_mask_loss
        rng = np.random.RandomState(seed)
        tokens_per_epoch = indexed.num_tokens
        epochs = max(1, -(-(num_samples * seq_length + 1) // max(tokens_per_epoch, 1)))
        docs = np.concatenate([rng.permutation(len(indexed)) for _ in range(epochs)])
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
