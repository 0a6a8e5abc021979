"""``document``: one document per item; contiguous block per rank, or a seeded shuffle dealt out
round-robin (optimus_dl/modules/data/datasets/strategies/document.py:15-85)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import numpy as np

from ....core.registry import RegistryConfigStrict
from . import register_strategy
from .base import BaseStrategy


@dataclass
class DocumentStrategyConfig(RegistryConfigStrict):
    shuffle: bool = False


@register_strategy("document", DocumentStrategyConfig)
class DocumentStrategy(BaseStrategy):
    """``indices`` (this rank's documents, in visiting order) and ``ptr`` (how many were visited) are the state, under
    the reference's names. Unshuffled, rank ``r`` of ``W`` gets documents ``[r * (n // W), (r + 1) * (n // W))`` and
    the last rank also the remainder; shuffled, a permutation drawn from the corpus-wide seed is dealt out
    round-robin."""

    indices: np.ndarray | None = None
    ptr: int = 0

    def _order(self) -> np.ndarray:
        n = len(self.doc_lens)
        if self.cfg is not None and self.cfg.shuffle:
            perm = np.random.default_rng(self.seed_base()).permutation(n)
            return perm[self.rank::self.world_size]
        per = n // self.world_size
        end = per * (self.rank + 1) if self.rank < self.world_size - 1 else n
        return np.arange(per * self.rank, end, dtype=np.int64)

    def reset(self, state: dict | None) -> None:
        self.indices = self._order()
        self.ptr = int(state.get("ptr", state.get("pos", 0))) if state else 0      # "pos": this package's earlier key

    def get_state(self) -> dict[str, Any]:
        return {"ptr": self.ptr, "rank": self.rank}

    def next_segments(self) -> list[tuple[int, int, int]]:
        if self.ptr >= len(self.indices):
            raise StopIteration
        d = int(self.indices[self.ptr])
        self.ptr += 1
        return [(d, 0, int(self.doc_lens[d]))]
