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
    seed: int = 0


@register_strategy("concat_random", ConcatRandomStrategyConfig)
class ConcatRandomStrategy(BaseStrategy):
    def initialize(self, doc_lens: np.ndarray) -> None:
        self.doc_lens = np.asarray(doc_lens, dtype=np.int64)
        self.cum = np.concatenate([[0], np.cumsum(self.doc_lens)])
        self.total = int(self.cum[-1])
        self.reset(None)

    def reset(self, state: dict | None) -> None:
        rng = np.random.default_rng(int(self.cfg.seed))   # identical on every rank
        cs = int(self.cfg.chunk_size)
        self.offset = int(rng.integers(0, cs)) if (self.cfg.random_offset and self.total > cs) else 0
        n_chunks = max(0, (self.total - self.offset) // cs)
        perm = rng.permutation(n_chunks)
        self.my_chunks = perm[self.rank::self.world_size]
        self.pos = int(state["pos"]) if state else 0

    def get_state(self) -> dict[str, Any]:
        return {"pos": self.pos}

    def next_segments(self) -> list[tuple[int, int, int]]:
        if self.pos >= len(self.my_chunks):
            raise StopIteration
        cs = int(self.cfg.chunk_size)
        start = self.offset + int(self.my_chunks[self.pos]) * cs
        end = start + cs
        self.pos += 1
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
