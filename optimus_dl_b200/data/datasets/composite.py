"""``composite``: weighted mixture of named datasets
(optimus_dl/modules/data/datasets/composite.py:27-403).

Indices are drawn from a seeded multinomial in blocks of 1000; the generator state before the current block
and the offset into it are checkpointed, so resume continues the exact same sequence. A
dataset that runs out is either restarted (``cycle``) or disabled; ``stop_criteria`` decides when the
mixture itself ends. ``strict_load`` makes resume fail if the set of datasets changed.
"""

from __future__ import annotations

import copy
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
    """Names drawn from a seeded multinomial in blocks of ``BLOCK``. What is checkpointed is the generator state from
    BEFORE the current block was drawn plus the offset into it, so a restored sampler redraws the same block and
    continues inside it; switching a dataset off discards the rest of the block (the next draw uses the new weights).
    Generator seeding, draw and state keys are those of optimus_dl/modules/data/datasets/composite.py:78-199."""

    BLOCK = 1000

    def __init__(self, weights: dict[str, float], seed: int, epoch: int = 0, state: dict | None = None):
        self.names = list(weights)
        self.original = torch.tensor([float(weights[n]) for n in self.names], dtype=torch.float64)
        self.weights = self.original.clone()
        self.gen = torch.Generator()
        self.gen.manual_seed(_epoch_seed(seed, epoch))
        self.snapshot = self.gen.get_state()
        self.offset = 0
        if state is not None:
            self.gen.set_state(state["g_state"])
            self.snapshot = self.gen.get_state()
            self.offset = int(state["offset"])
            if "weights" in state:
                self.weights = torch.as_tensor(state["weights"], dtype=torch.float64).clone()
        self.block = self._draw()

    def _draw(self) -> list[int]:
        if float(self.weights.sum()) == 0.0:
            return []
        self.snapshot = self.gen.get_state()
        return torch.multinomial(self.weights, self.BLOCK, replacement=True, generator=self.gen).tolist()

    def set_active(self, name: str, active: bool) -> None:
        i = self.names.index(name)
        self.weights[i] = self.original[i] if active else 0.0
        self.block, self.offset = [], 0

    def disable(self, name: str) -> None:
        self.set_active(name, False)

    def any_active(self) -> bool:
        return bool((self.weights > 0).any())

    def next(self) -> str:
        if self.offset >= len(self.block):
            self.block, self.offset = self._draw(), 0
            if not self.block:
                raise StopIteration
        self.offset += 1
        return self.names[self.block[self.offset - 1]]

    __next__ = next

    def __iter__(self):
        return self

    def state_dict(self) -> dict[str, Any]:
        return {"g_state": self.snapshot, "offset": self.offset, "weights": self.weights}

    state = state_dict


@register_dataset("composite", CompositeDatasetConfig)
class CompositeDataset(BaseDataset):
    """State keys (optimus_dl/modules/data/datasets/composite.py:217-221, 387-403): ``datasets_exhausted`` (name ->
    bool), ``dataset_node_states``, ``epoch``, ``num_yielded``, ``weighted_sampler_state``; ``cycles`` (how often each
    dataset was restarted) is this package's addition."""

    def __init__(self, cfg, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        super().__init__(cfg, rank, world_size, seed)
        self.kwargs = dict(kwargs, rank=rank, world_size=world_size, seed=seed)
        self.entries = {name: cfg.datasets[name] for name in cfg.datasets}
        if not self.entries:
            raise ValueError("composite dataset needs at least one entry")
        if any(float(e.weight) < 0 for e in self.entries.values()):
            raise ValueError("Weights must be non-negative")
        self.datasets = {n: build_dataset(e.dataset, **self.kwargs) for n, e in self.entries.items()}
        sc = cfg.stop_criteria
        self.stop = sc if isinstance(sc, StopCriteria) else StopCriteria(str(sc).split(".")[-1])
        self._epoch = 0
        self._num_yielded = 0
        self.sampler: _WeightedSampler | None = None
        self._datasets_exhausted: dict[str, bool] = {}
        self.epochs = {n: 0 for n in self.entries}

    @property
    def weights(self) -> dict[str, float]:
        return {n: e.weight for n, e in self.entries.items()}

    @property
    def exhausted(self) -> set[str]:
        return {n for n, done in self._datasets_exhausted.items() if done}

    @property
    def _weighted_sampler(self) -> _WeightedSampler | None:
        return self.sampler

    def _new_sampler(self, state: dict | None = None) -> _WeightedSampler:
        return _WeightedSampler(self.weights, self.seed, epoch=self._epoch, state=state)

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        if initial_state is not None:
            node_states = initial_state.get("dataset_node_states", {})
            saved = set(node_states)
            if self.cfg.strict_load and saved != set(self.datasets):
                raise ValueError(f"Strict load enabled. Mismatch in datasets.\nConfig: {sorted(self.datasets)}\n"
                                 f"State: {sorted(saved)}")
            self._num_yielded = int(initial_state.get("num_yielded", 0))
            self._epoch = int(initial_state.get("epoch", 0))
            self._datasets_exhausted = dict(initial_state.get("datasets_exhausted", dict.fromkeys(self.datasets, False)))
            self.epochs = dict(initial_state.get("cycles", {n: 0 for n in self.entries}))
            # the sampler's state only means something for the same set of datasets
            self.sampler = self._new_sampler(initial_state.get("weighted_sampler_state") if saved == set(self.datasets)
                                             else None)
            for n, ds in self.datasets.items():
                ds.reset(node_states[n]) if n in node_states else ds.reset()
        else:
            self._num_yielded = self._epoch = 0
            self.sampler = self._new_sampler()
            self._datasets_exhausted = dict.fromkeys(self.datasets, False)
            self.epochs = {n: 0 for n in self.entries}
            for ds in self.datasets.values():
                ds.reset()

    def get_state(self) -> dict[str, Any]:
        return copy.deepcopy({
            "datasets_exhausted": self._datasets_exhausted,
            "dataset_node_states": {n: ds.state_dict() for n, ds in self.datasets.items()},
            "epoch": self._epoch, "num_yielded": self._num_yielded,
            "weighted_sampler_state": self.sampler.state_dict() if self.sampler is not None else None,
            "cycles": self.epochs})

    def _check_stop(self) -> None:
        """Stop rules of optimus_dl/modules/data/datasets/composite.py:328-338: a dataset that cycles never counts as
        exhausted; ``cycle_forever`` never stops; otherwise the stream ends when every dataset is exhausted, or, with
        ``first_dataset_exhausted``, when any is."""
        if self.stop == StopCriteria.CYCLE_FOREVER:
            return
        if self._datasets_exhausted and all(self._datasets_exhausted.values()):
            raise StopIteration
        if self.stop == StopCriteria.FIRST_DATASET_EXHAUSTED and any(self._datasets_exhausted.values()):
            raise StopIteration

    def next(self) -> Any:
        if self.sampler is None:
            self.reset()
        while True:
            self._check_stop()
            try:
                name = next(self.sampler)
            except StopIteration as err:
                raise RuntimeError("every dataset is exhausted and none of them cycles") from err
            try:
                item = next(self.datasets[name])
                self._num_yielded += 1
                return item
            except StopIteration:
                if self.entries[name].cycle:
                    self.epochs[name] = self.epochs.get(name, 0) + 1
                    self.datasets[name].reset()
                    try:
                        item = next(self.datasets[name])
                        self._num_yielded += 1
                        return item
                    except StopIteration as err:
                        raise RuntimeError(f"dataset '{name}' yields nothing after the reset that should cycle it") from err
                self._datasets_exhausted[name] = True
                self.sampler.set_active(name, False)
