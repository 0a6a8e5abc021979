"""``concat_random``: treat the corpus as one token stream, cut it into fixed-size chunks starting at
a random global offset, visit the chunks in a seeded permutation, rank-strided
(optimus_dl/modules/data/datasets/strategies/concat_random.py:15-171). Every token between the
offset and the last full chunk is seen exactly once per epoch across all ranks."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import numpy as np

from ....core.registry import RegistryConfigStrict
from . import register_strategy
from .base import BaseStrategy


@dataclass
class ConcatRandomStrategyConfig(RegistryConfigStrict):
    chunk_size: int = 2048
    random_offset: bool = True
    seed: int | None = None      # overrides the dataset's seed for the chunk order (not a reference field)


@register_strategy("concat_random", ConcatRandomStrategyConfig)
class ConcatRandomStrategy(BaseStrategy):
    """State and attributes under the reference's names: ``global_offset``, ``my_chunk_indices``, ``chunk_ptr``;
    ``get_state`` returns ``chunk_ptr``, ``seed`` and ``rank``. The generator is consumed in the reference's order
    (offset first, whenever ``random_offset`` is set, then the permutation), so one seed gives one schedule in both
    code bases."""

    global_offset: int = 0
    my_chunk_indices: np.ndarray | None = None
    chunk_ptr: int = 0

    def initialize(self, doc_lens: np.ndarray) -> None:
        self.doc_lens = np.asarray(doc_lens, dtype=np.int64)
        self.cum = np.concatenate([[0], np.cumsum(self.doc_lens)])
        self.total = int(self.cum[-1])
        self.reset(None)

    def _schedule_seed(self) -> int:
        own = self.cfg.get("seed") if hasattr(self.cfg, "get") else getattr(self.cfg, "seed", None)
        return int(own) if own is not None else self.seed_base()

    def reset(self, state: dict | None) -> None:
        seed = int(state["seed"]) if state and state.get("seed") is not None else self._schedule_seed()
        self.schedule_seed = seed
        rng = np.random.default_rng(seed)                   # identical on every rank
        cs = int(self.cfg.chunk_size)
        self.global_offset = int(rng.integers(0, cs)) if self.cfg.random_offset else 0
        n_chunks = max(0, (self.total - self.global_offset) // cs)
        perm = rng.permutation(n_chunks)
        self.my_chunk_indices = perm[self.rank::self.world_size]
        self.chunk_ptr = int(state.get("chunk_ptr", state.get("pos", 0))) if state else 0

    def get_state(self) -> dict[str, Any]:
        return {"chunk_ptr": self.chunk_ptr, "seed": self.schedule_seed, "rank": self.rank}

    def next_segments(self) -> list[tuple[int, int, int]]:
        if self.chunk_ptr >= len(self.my_chunk_indices):
            raise StopIteration
        cs = int(self.cfg.chunk_size)
        start = self.global_offset + int(self.my_chunk_indices[self.chunk_ptr]) * cs
        end = start + cs
        self.chunk_ptr += 1
        segs = []
        d = int(np.searchsorted(self.cum, start, side="right") - 1)
        while start < end:
            d_end = int(self.cum[d + 1])
            take = min(end, d_end)
            if take > start:
                segs.append((d, start - int(self.cum[d]), take - int(self.cum[d])))
            start = take
            d += 1
        return segs


# the reference's class names for this strategy
ConcatAndChunkFullRandom = ConcatRandomStrategy
ConcatAndChunkFullRandomConfig = ConcatRandomStrategyConfig
