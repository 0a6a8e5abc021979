"""``composite``: weighted mixture of named datasets
(optimus_dl/modules/data/datasets/composite.py:27-403).

Indices are drawn from a seeded multinomial in blocks of 1000; the generator state and the unread
part of the current block are checkpointed, so resume continues the exact same sequence. A
dataset that runs out is either restarted (``cycle``) or disabled; ``stop_criteria`` decides when the
mixture itself ends. ``strict_load`` makes resume fail if the set of datasets changed.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any

import torch

from ...core.registry import RegistryConfigStrict
from . import build_dataset, register_dataset
from .base import BaseDataset


class StopCriteria(str, enum.Enum):
    FIRST_DATASET_EXHAUSTED = "FIRST_DATASET_EXHAUSTED"
    ALL_DATASETS_EXHAUSTED = "ALL_DATASETS_EXHAUSTED"
    CYCLE_FOREVER = "CYCLE_FOREVER"


@dataclass
class DatasetConfig:
    dataset: Any = "???"
    weight: float = 1.0
    cycle: bool = True


@dataclass
class CompositeDatasetConfig(RegistryConfigStrict):
    datasets: dict[str, DatasetConfig] = field(default_factory=dict)
    strict_load: bool = True
    stop_criteria: StopCriteria = StopCriteria.CYCLE_FOREVER


def _epoch_seed(seed: int, epoch: int) -> int:
    g = torch.Generator()
    g.manual_seed(int(seed) + int(epoch) * 10000)
    return int(torch.randint(0, 2**32, (1,), generator=g).item())


class _WeightedSampler:
    BLOCK = 1000

    def __init__(self, weights: dict[str, float], seed: int, epoch: int = 0, state: dict | None = None):
        self.names = list(weights)
        self.original = torch.tensor([float(weights[n]) for n in self.names], dtype=torch.float64)
        self.weights = self.original.clone()
        self.gen = torch.Generator()
        self.gen.manual_seed(_epoch_seed(seed, epoch))
        self.block: list[int] = []
        if state is not None:
            self.gen.set_state(state["gen"])
            self.block = list(state["block"])
            self.weights = torch.tensor(state["weights"], dtype=torch.float64)

    def disable(self, name: str) -> None:
        self.weights[self.names.index(name)] = 0.0
        self.block = [i for i in self.block if self.weights[i] > 0]

    def any_active(self) -> bool:
        return bool((self.weights > 0).any())

    def next(self) -> str:
        if not self.block:
            idx = torch.multinomial(self.weights / self.weights.sum(), self.BLOCK, replacement=True, generator=self.gen)
            self.block = idx.tolist()
        return self.names[self.block.pop(0)]

    def state(self) -> dict[str, Any]:
        return {"gen": self.gen.get_state(), "block": list(self.block), "weights": self.weights.tolist()}


@register_dataset("composite", CompositeDatasetConfig)
class CompositeDataset(BaseDataset):
    def __init__(self, cfg, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        super().__init__(cfg, rank, world_size, seed)
        self.kwargs = dict(kwargs, rank=rank, world_size=world_size, seed=seed)
        self.entries = {name: cfg.datasets[name] for name in cfg.datasets}
        if not self.entries:
            raise ValueError("composite dataset needs at least one entry")
        self.datasets = {n: build_dataset(e.dataset, **self.kwargs) for n, e in self.entries.items()}
        sc = cfg.stop_criteria
        self.stop = sc if isinstance(sc, StopCriteria) else StopCriteria(str(sc).split(".")[-1])
        self.sampler = _WeightedSampler({n: e.weight for n, e in self.entries.items()}, seed)
        self.exhausted: set[str] = set()
        self.epochs = {n: 0 for n in self.entries}

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        weights = {n: e.weight for n, e in self.entries.items()}
        if initial_state:
            saved = set(initial_state["datasets"])
            if self.cfg.strict_load and saved != set(self.datasets):
                raise ValueError(f"composite dataset state has {sorted(saved)} but config has {sorted(self.datasets)}")
            self.sampler = _WeightedSampler(weights, self.seed, state=initial_state["sampler"])
            self.exhausted = set(initial_state.get("exhausted", []))
            self.epochs = dict(initial_state.get("epochs", {n: 0 for n in self.entries}))
            for n, ds in self.datasets.items():
                ds.reset(initial_state["datasets"].get(n))
        else:
            self.sampler = _WeightedSampler(weights, self.seed)
            self.exhausted = set()
            self.epochs = {n: 0 for n in self.entries}
            for ds in self.datasets.values():
                ds.reset()

    def get_state(self) -> dict[str, Any]:
        return {"sampler": self.sampler.state(), "exhausted": sorted(self.exhausted), "epochs": dict(self.epochs),
                "datasets": {n: ds.state_dict() for n, ds in self.datasets.items()}}

    def _check_stop(self) -> None:
        """Stop rules of optimus_dl/modules/data/datasets/composite.py:328-338: a dataset that cycles never counts as
        exhausted; ``cycle_forever`` never stops; otherwise the stream ends when every dataset is exhausted, or, with
        ``first_dataset_exhausted``, when any is."""
        if self.stop == StopCriteria.CYCLE_FOREVER:
            return
        if self.exhausted == set(self.datasets):
            raise StopIteration
        if self.stop == StopCriteria.FIRST_DATASET_EXHAUSTED and self.exhausted:
            raise StopIteration

    def next(self) -> Any:
        while True:
            self._check_stop()
            if not self.sampler.any_active():
                raise RuntimeError("every dataset is exhausted and none of them cycles")
            name = self.sampler.next()
            try:
                return next(self.datasets[name])
            except StopIteration:
                if self.entries[name].cycle:
                    self.epochs[name] += 1
                    self.datasets[name].reset()
                    try:
                        return next(self.datasets[name])
                    except StopIteration as err:
                        raise RuntimeError(f"dataset '{name}' yields nothing after the reset that should cycle it") from err
                self.exhausted.add(name)
                self.sampler.disable(name)
