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
    def _order(self) -> np.ndarray:
        n = len(self.doc_lens)
        if self.cfg is not None and self.cfg.shuffle:
            perm = np.random.default_rng(self.seed_base()).permutation(n)
            return perm[self.rank::self.world_size]
        per = (n + self.world_size - 1) // self.world_size
        return np.arange(self.rank * per, min(n, (self.rank + 1) * per))

    def seed_base(self) -> int:
        return int(getattr(self, "global_seed", 0))

    def reset(self, state: dict | None) -> None:
        self.order = self._order()
        self.pos = int(state["pos"]) if state else 0

    def get_state(self) -> dict[str, Any]:
        return {"pos": self.pos}

    def next_segments(self) -> list[tuple[int, int, int]]:
        if self.pos >= len(self.order):
            raise StopIteration
        d = int(self.order[self.pos])
        self.pos += 1
        return [(d, 0, int(self.doc_lens[d]))]
