"""Synthetic (mock) token batches: uniform random ids from a seed, labels = inputs shifted by
one. Equivalent of the reference's ``--mock-data`` / ``MockGPTDataset`` path
(loongforge/train/pretrain/pretrain_llm.py:198-229). Batches are produced on the HOST in pinned
memory so that the training step includes a real host-to-device copy."""
from __future__ import annotations

from typing import Dict, Iterator, Optional

import torch


class SyntheticTokenDataset:
    def __init__(self, vocab_size: int, seq_length: int, seed: int = 1234, num_samples: int = 1 << 30):
        self.vocab_size, self.seq_length, self.seed, self.num_samples = vocab_size, seq_length, seed, num_samples

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        g = torch.Generator()
        g.manual_seed(self.seed * 1_000_003 + idx)
        t = torch.randint(0, self.vocab_size, (self.seq_length + 1,), generator=g, dtype=torch.int64)
        return {"tokens": t[:-1], "labels": t[1:]}


def synthetic_batch_iterator(vocab_size: int, seq_length: int, micro_batch_size: int, *, dp_rank: int = 0,
                             dp_size: int = 1, seed: int = 1234, pin_memory: Optional[bool] = None,
                             start_sample: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Infinite iterator of micro-batches for one data-parallel rank. Sample `i` of the global
    stream goes to rank ``(i // micro_batch_size) % dp_size`` so that the union over ranks is
    independent of the parallel layout."""
    ds = SyntheticTokenDataset(vocab_size, seq_length, seed)
    pin = torch.cuda.is_available() if pin_memory is None else pin_memory
    pos = torch.arange(seq_length, dtype=torch.int64).unsqueeze(0).expand(micro_batch_size, -1).contiguous()
    step = 0
    while True:
        base = start_sample + (step * dp_size + dp_rank) * micro_batch_size
        items = [ds[base + j] for j in range(micro_batch_size)]
        batch = {
            "tokens": torch.stack([it["tokens"] for it in items]),
            "labels": torch.stack([it["labels"] for it in items]),
            "loss_mask": torch.ones(micro_batch_size, seq_length, dtype=torch.float32),
            "position_ids": pos.clone(),
        }
        if pin:
            batch = {k: v.pin_memory() for k, v in batch.items()}
        batch["num_valid_tokens"] = micro_batch_size * seq_length
        yield batch
        step += 1
