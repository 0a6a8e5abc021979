"""``synthetic_tokens``: uniform-random token ids, the data source of the benchmark configs.

Not part of the reference (it reads real corpora); the benchmark protocol asks for synthetic
uniform token ids of a given shape. Each item is one document ``{"input_ids": int64[length]}``;
the stream is a pure function of ``(seed, rank, position)`` so resume is exact.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import numpy as np

from ...core.registry import RegistryConfigStrict
from . import register_dataset
from .base import BaseDataset


@dataclass
class SyntheticTokensConfig(RegistryConfigStrict):
    vocab_size: int = 50257
    length: int = 1025                 # tokens per document (fixed) unless mean_length is set
    mean_length: float | None = None   # exponential document lengths with this mean
    min_length: int = 32
    max_length: int | None = None
    num_documents: int | None = None   # None = endless
    seed: int = 0


@register_dataset("synthetic_tokens", SyntheticTokensConfig)
class SyntheticTokensDataset(BaseDataset):
    def __init__(self, cfg, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        super().__init__(cfg, rank, world_size, seed)
        self.position = 0

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self.position = int(initial_state["position"]) if initial_state else 0

    def get_state(self) -> dict[str, Any]:
        return {"position": self.position}

    def next(self) -> dict[str, Any]:
        cfg = self.cfg
        if cfg.num_documents is not None and self.position >= cfg.num_documents:
            raise StopIteration
        rng = np.random.default_rng([int(cfg.seed), int(self.seed) % (2**32), self.rank, self.position])
        if cfg.mean_length is not None:
            n = max(int(cfg.min_length), int(rng.exponential(cfg.mean_length)))
            if cfg.max_length is not None:
                n = min(n, int(cfg.max_length))
        else:
            n = int(cfg.length)
        self.position += 1
        return {"input_ids": rng.integers(0, cfg.vocab_size, size=n, dtype=np.int64)}
