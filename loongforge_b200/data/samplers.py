"""Samplers and iterators of the SFT / ChunkPipe data path: a group sampler that balances cost across data-parallel
ranks (longest-processing-time partition) and packs greedily within a rank, and cyclic iterators whose position can be
saved and restored (reference: loongforge/train/sft/utils.py:330-972 group sampler, :1193-1464 savable iterators)."""
from __future__ import annotations

from typing import Dict, Iterator, List, Sequence

import numpy as np

from .packing import lpt_partition, pack_first_fit_decreasing


class BalancedGroupSampler:
    """Each step takes `group_size` samples (in a seeded shuffled order), splits them over the DP ranks so that the
    summed cost (``len^2`` by default: attention dominates long sequences) is even, and returns this rank's share packed
    into sequences of at most `capacity` tokens."""

    def __init__(self, lengths: Sequence[int], group_size: int, dp_size: int, dp_rank: int, capacity: int,
                 seed: int = 0, cost=lambda n: float(n) * float(n)):
        self.lengths, self.G, self.dp, self.rank, self.cap = list(lengths), group_size, dp_size, dp_rank, capacity
        self.seed, self.cost = seed, cost
        self.epoch, self.cursor = 0, 0
        self._order = self._shuffle()

    def _shuffle(self) -> np.ndarray:
        return np.random.default_rng(self.seed + self.epoch).permutation(len(self.lengths))

    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "cursor": self.cursor}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.epoch, self.cursor = sd["epoch"], sd["cursor"]
        self._order = self._shuffle()

    def __iter__(self) -> Iterator[List[List[int]]]:
        while True:
            if self.cursor + self.G > len(self._order):
                self.epoch, self.cursor = self.epoch + 1, 0
                self._order = self._shuffle()
            group = [int(i) for i in self._order[self.cursor:self.cursor + self.G]]
            self.cursor += self.G
            parts = lpt_partition([self.cost(self.lengths[i]) for i in group], self.dp)
            mine = [group[j] for j in parts[self.rank]]
            packs = pack_first_fit_decreasing([min(self.lengths[i], self.cap) for i in mine], self.cap)
            yield [[mine[j] for j in p] for p in packs]


class SavableCyclicIterator:
    """Cycles over an indexable dataset forever in a seeded order; `state_dict` captures (epoch, position) so that a
    resumed run continues with the very next sample."""

    def __init__(self, dataset, seed: int = 0, shuffle: bool = True):
        self.ds, self.seed, self.shuffle = dataset, seed, shuffle
        self.epoch, self.pos = 0, 0
        self._perm = self._order()

    def _order(self):
        n = len(self.ds)
        return np.random.default_rng(self.seed + self.epoch).permutation(n) if self.shuffle else np.arange(n)

    def __iter__(self):
        return self

    def __next__(self):
        if self.pos >= len(self._perm):
            self.epoch, self.pos = self.epoch + 1, 0
            self._perm = self._order()
        item = self.ds[int(self._perm[self.pos])]
        self.pos += 1
        return item

    def state_dict(self):
        return {"epoch": self.epoch, "pos": self.pos}

    def load_state_dict(self, sd):
        self.epoch, self.pos = sd["epoch"], sd["pos"]
        self._perm = self._order()


class PrefetchIterator:
    """Runs a batch iterator in a background thread and keeps up to ``depth`` batches ready, so that tokenisation, image
    decoding and packing overlap the training step (``--num-workers``: depth = 2 x workers; one producer thread, since the
    iterators are stateful generators). An exception in the producer is raised in the consumer at the same position.
    ``close()`` stops the thread; batches prepared ahead are dropped — resuming goes by the trainer's sample counter."""

    _END = object()

    def __init__(self, iterator, depth: int = 4):
        import queue
        import threading
        self.q: "queue.Queue" = queue.Queue(maxsize=max(depth, 1))
        self._stop = threading.Event()
        self._it = iterator

        def work():
            try:
                for item in self._it:
                    while not self._stop.is_set():
                        try:
                            self.q.put(item, timeout=0.1)
                            break
                        except queue.Full:
                            continue
                    if self._stop.is_set():
                        return
                self.q.put(self._END)
            except BaseException as e:  # noqa: BLE001 - handed to the consumer
                self.q.put(e)

        self.thread = threading.Thread(target=work, daemon=True, name="data-prefetch")
        self.thread.start()

    def __iter__(self):
        return self

    def __next__(self):
        item = self.q.get()
        if item is self._END:
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        return item

    def close(self):
        self._stop.set()
        try:
            while True:
                self.q.get_nowait()
        except Exception:  # noqa: BLE001 - queue.Empty
            pass
        self.thread.join(timeout=2.0)
