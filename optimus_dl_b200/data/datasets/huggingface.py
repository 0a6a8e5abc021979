"""``huggingface_dataset``: Hugging Face ``datasets`` streams, split by node across ranks, resumable
through the stream's own ``state_dict`` or by skipping (optimus_dl/modules/data/datasets/huggingface.py:21-131)."""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from ...core.registry import RegistryConfigStrict
from . import register_dataset
from .base import BaseDataset


@dataclass
class HuggingFaceDatasetConfig(RegistryConfigStrict):
    dataset_load_kwargs: dict = "???"  # type: ignore[assignment]


def __getattr__(name: str) -> Any:
    """``load_dataset`` is a module-level name (callers can substitute it) that imports the optional and
    slow-to-import ``datasets`` package on first use only."""
    if name == "load_dataset":
        from datasets import load_dataset

        return load_dataset
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


@register_dataset("huggingface_dataset", HuggingFaceDatasetConfig)
class HuggingFaceDataset(BaseDataset):
    def __init__(self, cfg, rank: int = 0, world_size: int = 1, **kwargs: Any):
        super().__init__(cfg, rank, world_size, kwargs.get("seed", 0))
        self.position = 0
        self._iter = None
        self._ds = None

    def _open(self):
        load_dataset = globals().get("load_dataset") or __getattr__("load_dataset")
        kw = dict(self.cfg.dataset_load_kwargs)
        kw.setdefault("streaming", True)
        ds = load_dataset(**kw)
        if self.world_size > 1:
            from datasets.distributed import split_dataset_by_node

            ds = split_dataset_by_node(ds, rank=self.rank, world_size=self.world_size)
        return ds

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self._ds = self._open()
        self.position = 0
        if initial_state:
            assert initial_state.get("rank", self.rank) == self.rank and \
                initial_state.get("world_size", self.world_size) == self.world_size, \
                "huggingface_dataset must be resumed with the same rank and world size"
            self.position = int(initial_state.get("position", 0))
            hf_state = initial_state.get("dataset_state", initial_state.get("hf_state"))    # "hf_state": earlier key
            if hf_state is not None and hasattr(self._ds, "load_state_dict"):
                self._ds.load_state_dict(hf_state)
            elif self.position:
                self._ds = self._ds.skip(self.position) if hasattr(self._ds, "skip") else self._ds.select(
                    range(self.position, len(self._ds)))
        self._iter = iter(self._ds)

    def get_state(self) -> dict[str, Any]:
        """Keys of optimus_dl/modules/data/datasets/huggingface.py:58-72."""
        st: dict[str, Any] = {"cfg": copy.deepcopy(self.cfg), "dataset_state": None, "world_size": self.world_size,
                              "rank": self.rank, "position": self.position}
        if self._ds is not None and hasattr(self._ds, "state_dict"):
            try:
                st["dataset_state"] = copy.deepcopy(self._ds.state_dict())
            except Exception:
                pass
        return st

    def next(self) -> Any:
        if self._iter is None:
            self.reset()
        item = next(self._iter)
        self.position += 1
        return item
