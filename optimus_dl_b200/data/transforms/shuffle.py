"""``shuffle``: seeded shuffle buffer; the generator is seeded with ``seed + rank * 41`` and its state is part of
the checkpoint
(optimus_dl/modules/data/transforms/shuffle.py:17-121)."""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

import numpy as np
from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform, adopt_saved_cfg


@dataclass
class ShuffleTransformConfig(RegistryConfigStrict):
    buffer_size: int = 1024


class ShuffleNode(BaseNode):
    """Fill a buffer of ``buffer_size`` items, then hand out a uniformly drawn one per call (the others keep their
    order). Generator (numpy ``default_rng``), draw (``integers(0, len(buffer))``) and state keys are the
    reference's, so one seed gives one stream in both code bases and checkpoints of this node are interchangeable."""

    def __init__(self, node: BaseNode, cfg: Any, rank: int = 0, seed: int = 0):
        super().__init__()
        self.node, self.cfg, self.rank = node, cfg, int(rank)
        self._default_seed = int(seed) + self.rank * 41
        self.rng = np.random.default_rng(self._default_seed)
        self.buffer: list = []
        self.terminated = False

    @property
    def buffer_size(self) -> int:
        return int(self.cfg.buffer_size)

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self.buffer, self.terminated = [], False
        self.rng = np.random.default_rng(self._default_seed)
        if initial_state:
            self.buffer = copy.deepcopy(initial_state["buffer"])
            self.cfg = adopt_saved_cfg(self.cfg, initial_state.get("cfg"))
            self.rng.bit_generator.state = initial_state["rng_state"]
            self.terminated = bool(initial_state["terminated"])
            assert initial_state.get("rank", self.rank) == self.rank, "shuffle state belongs to another rank"
            self.node.reset(initial_state["source_state"])
        else:
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        return copy.deepcopy({"buffer": self.buffer, "cfg": self.cfg, "source_state": self.node.state_dict(),
                              "rng_state": self.rng.bit_generator.state, "terminated": self.terminated,
                              "rank": self.rank})

    def next(self) -> Any:
        while not self.terminated and len(self.buffer) < self.buffer_size:
            try:
                self.buffer.append(next(self.node))
            except StopIteration:
                self.terminated = True
        if not self.buffer:
            raise StopIteration
        return self.buffer.pop(int(self.rng.integers(0, len(self.buffer))))


@register_transform("shuffle", ShuffleTransformConfig)
class ShuffleTransform(BaseTransform):
    def __init__(self, cfg, rank: int = 0, seed: int = 0, **kwargs: Any):
        super().__init__(cfg)
        self.rank, self.seed = int(rank), int(seed)

    def build(self, source: BaseNode) -> BaseNode:
        return ShuffleNode(source, self.cfg, rank=self.rank, seed=self.seed)


ShuffleTransformNode = ShuffleNode   # the reference's name
