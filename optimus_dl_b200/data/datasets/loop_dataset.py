"""``loop``: restart the inner dataset whenever it is exhausted
(optimus_dl/modules/data/datasets/loop_dataset.py:20-95)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ...core.registry import RegistryConfig
from . import build_dataset, register_dataset
from .base import BaseDataset


@dataclass
class LoopDatasetConfig(RegistryConfig):
    inner: Any = None


@register_dataset("loop", LoopDatasetConfig)
class LoopDataset(BaseDataset):
    def __init__(self, cfg, **kwargs: Any):
        super().__init__(cfg, **{k: kwargs[k] for k in ("rank", "world_size", "seed") if k in kwargs})
        self.kwargs = kwargs
        self.inner = build_dataset(cfg.inner, **kwargs)
        self.epoch = 0

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        if initial_state:
            assert initial_state.get("rank", self.rank) == self.rank and \
                initial_state.get("world_size", self.world_size) == self.world_size, \
                "loop must be resumed with the same rank and world size"
            self.epoch = initial_state.get("epoch", 0)
            self.inner.reset(initial_state.get("inner_state"))
        else:
            self.epoch = 0
            self.inner.reset()

    def get_state(self) -> dict[str, Any]:
        return {"rank": self.rank, "world_size": self.world_size, "epoch": self.epoch, "inner_state": self.inner.state_dict()}

    def next(self) -> Any:
        try:
            return next(self.inner)
        except StopIteration:
            self.epoch += 1
            self.inner = build_dataset(self.cfg.inner, **self.kwargs)
            self.inner.reset()
            try:
                return next(self.inner)
            except StopIteration:
                raise RuntimeError("loop: inner dataset is empty") from None
