"""Strategy interface (optimus_dl/modules/data/datasets/strategies/base.py:18-63): given the document
lengths of the whole corpus, yield ``(doc_index, start, end)`` token ranges for this rank."""

from __future__ import annotations

from typing import Any

import numpy as np


class BaseStrategy:
    def __init__(self, cfg: Any = None, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        self.cfg, self.rank, self.world_size, self.seed = cfg, rank, world_size, seed
        self.doc_lens: np.ndarray | None = None

    def seed_base(self) -> int:
        """Seed of everything the ranks must agree on (permutations, offsets): the corpus-wide seed when the dataset
        was given one (``global_seed``), else the seed the strategy was built with, which is then expected to be the
        same on every rank, as in optimus_dl/modules/data/datasets/strategies/document.py:43-46."""
        g = getattr(self, "global_seed", None)
        return int(self.seed if g is None else g)

    def next_sample(self) -> list[tuple[int, tuple[int, int]]]:
        """The next item as ``[(doc_index, (start, end)), ...]``
        (the call form of optimus_dl/modules/data/datasets/strategies/base.py:45-55)."""
        return [(d, (a, b)) for d, a, b in self.next_segments()]

    def initialize(self, doc_lens: np.ndarray) -> None:
        self.doc_lens = np.asarray(doc_lens, dtype=np.int64)
        self.reset(None)

    def reset(self, state: dict | None) -> None:
        raise NotImplementedError

    def get_state(self) -> dict[str, Any]:
        raise NotImplementedError

    def next_segments(self) -> list[tuple[int, int, int]]:
        """Token ranges forming the next item; raises StopIteration at the end of this rank's share."""
        raise NotImplementedError
