"""Number of micro-batches per step, constant or ramped up
(Megatron's ``num_microbatches_calculator`` used at loongforge/train/training_utils.py:2687-2711)."""
from __future__ import annotations

from typing import Optional, Sequence


class MicrobatchCalculator:
    def __init__(self, global_batch_size: int, micro_batch_size: int, data_parallel_size: int,
                 rampup: Optional[Sequence[int]] = None):
        self.micro_batch_size = micro_batch_size
        self.dp = data_parallel_size
        self.final_gbs = global_batch_size
        self.rampup = rampup  # (start_gbs, increment, ramp_samples)
        per_step = micro_batch_size * data_parallel_size
        assert global_batch_size % per_step == 0, (
            f"global batch size {global_batch_size} is not divisible by micro batch size x data parallel "
            f"size ({micro_batch_size} x {data_parallel_size})")
        if rampup is not None:
            start, inc, samples = rampup
            assert (global_batch_size - start) % inc == 0
            self._n_inc = (global_batch_size - start) // inc
            self._samples_per_inc = samples / max(self._n_inc, 1)
        self.current_gbs = global_batch_size
        self.update(0)

    def update(self, consumed_samples: int, consistency_check: bool = True) -> None:
        if self.rampup is None:
            self.current_gbs = self.final_gbs
        else:
            start, inc, samples = self.rampup
            if consumed_samples > samples:
                self.current_gbs = self.final_gbs
            else:
                steps = int(consumed_samples / self._samples_per_inc)
                self.current_gbs = min(start + steps * inc, self.final_gbs)
        per_step = self.micro_batch_size * self.dp
        if consistency_check:
            assert self.current_gbs % per_step == 0
        self.num_microbatches = self.current_gbs // per_step

    def get(self) -> int:
        return self.num_microbatches
