"""``shuffle``: seeded reservoir-style shuffle buffer; the generator is seeded with
``seed + rank * 41`` and its state is part of the checkpoint
(optimus_dl/modules/data/transforms/shuffle.py:17-121)."""

from __future__ import annotations

import copy
import random
from dataclasses import dataclass
from typing import Any

from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform


@dataclass
class ShuffleTransformConfig(RegistryConfigStrict):
    buffer_size: int = 1024


class ShuffleNode(BaseNode):
    def __init__(self, node: BaseNode, buffer_size: int, seed: int):
        super().__init__()
        self.node, self.buffer_size, self.seed = node, int(buffer_size), seed
        self.rng = random.Random(seed)
        self.buffer: list = []
        self.exhausted = False

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        if initial_state:
            self.buffer = copy.deepcopy(initial_state["buffer"])
            self.rng.setstate(initial_state["rng"])
            self.exhausted = initial_state.get("exhausted", False)
            self.node.reset(initial_state["source_state"])
        else:
            self.buffer, self.exhausted = [], False
            self.rng = random.Random(self.seed)
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        return {"buffer": copy.deepcopy(self.buffer), "rng": self.rng.getstate(), "exhausted": self.exhausted,
                "source_state": self.node.state_dict()}

    def next(self) -> Any:
        while not self.exhausted and len(self.buffer) < self.buffer_size:
            try:
                self.buffer.append(next(self.node))
            except StopIteration:
                self.exhausted = True
        if not self.buffer:
            raise StopIteration
        i = self.rng.randrange(len(self.buffer))
        self.buffer[i], self.buffer[-1] = self.buffer[-1], self.buffer[i]
        return self.buffer.pop()


@register_transform("shuffle", ShuffleTransformConfig)
class ShuffleTransform(BaseTransform):
    def __init__(self, cfg, rank: int = 0, seed: int = 0, **kwargs: Any):
        super().__init__(cfg)
        self.seed = int(seed) + int(rank) * 41

    def build(self, source: BaseNode) -> BaseNode:
        return ShuffleNode(source, self.cfg.buffer_size, self.seed)


ShuffleTransformNode = ShuffleNode   # the reference's name
