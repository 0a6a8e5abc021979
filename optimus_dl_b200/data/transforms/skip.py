"""``skip_interleaved`` / ``skip_random``: drop items deterministically, e.g. to carve disjoint
subsets out of one stream (optimus_dl/modules/data/transforms/skip.py)."""

from __future__ import annotations

import random
from dataclasses import dataclass
from typing import Any

from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform


@dataclass
class SkipInterleavedConfig(RegistryConfigStrict):
    keep_every: int = 2      # keep one item out of this many
    offset: int = 0          # index (mod keep_every) of the kept item
    # the reference's spelling (optimus_dl/modules/data/transforms/skip.py:15-22): the first item is produced, then
    # ``skip_count`` items are dropped before each further one, i.e. keep_every = skip_count + 1 with offset 0
    skip_count: int | None = None


class SkipInterleavedNode(BaseNode):
    """``SkipInterleavedNode(node, cfg)`` or ``SkipInterleavedNode(node, keep_every, offset)``. ``counter`` is the number
    of source items consumed so far; the state stores it under ``counter``."""

    def __init__(self, node: BaseNode, keep_every: Any, offset: int = 0):
        super().__init__()
        self.cfg = None
        if not isinstance(keep_every, int):
            self.cfg = cfg = keep_every
            if cfg.skip_count is not None:
                keep_every, offset = int(cfg.skip_count) + 1, 0
            else:
                keep_every, offset = cfg.keep_every, cfg.offset
        self.node, self.keep_every, self.offset = node, max(1, int(keep_every)), int(offset)
        self.count = 0

    @property
    def counter(self) -> int:
        return self.count

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        if initial_state:
            self.count = initial_state["counter"] if "counter" in initial_state else initial_state["count"]
            self.node.reset(initial_state["source_state"])
        else:
            self.count = 0
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        return {"counter": self.count, "source_state": self.node.state_dict()}

    def next(self) -> Any:
        while True:
            item = next(self.node)
            keep = self.count % self.keep_every == self.offset % self.keep_every
            self.count += 1
            if keep:
                return item


@register_transform("skip_interleaved", SkipInterleavedConfig)
class SkipInterleaved(BaseTransform):
    def build(self, source: BaseNode) -> BaseNode:
        return SkipInterleavedNode(source, self.cfg)


@dataclass
class SkipRandomConfig(RegistryConfigStrict):
    keep_probability: float = 0.5
    seed: int = 0
    invert: bool = False     # keep exactly the items the non-inverted transform drops
    # the reference's spelling (optimus_dl/modules/data/transforms/skip.py:85-92): probability that an item is dropped;
    # an item is then dropped exactly when the draw is below it, as there
    probability: float | None = None


class SkipRandomNode(BaseNode):
    """``SkipRandomNode(node, cfg, seed=...)`` or ``SkipRandomNode(node, keep_probability, seed, invert)``."""

    def __init__(self, node: BaseNode, p: Any, seed: int | None = None, invert: bool = False):
        super().__init__()
        self.cfg = None
        self.drop_below: float | None = None     # set when configured through ``probability``
        if not isinstance(p, (int, float)):
            self.cfg = cfg = p
            p, invert = cfg.keep_probability, cfg.invert
            seed = cfg.seed if seed is None else seed
            if cfg.probability is not None:
                self.drop_below = float(cfg.probability)
        self.node, self.p, self.seed, self.invert = node, float(p), int(seed or 0), bool(invert)
        self.rng = random.Random(self.seed)

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        if initial_state:
            st = initial_state.get("rng_state", initial_state.get("rng"))      # "rng": this package's earlier key
            if st is not None:
                self.rng.setstate(tuple(tuple(x) if isinstance(x, list) else x for x in st))
            self.node.reset(initial_state["source_state"])
        else:
            self.rng = random.Random(self.seed)
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        return {"rng_state": self.rng.getstate(), "source_state": self.node.state_dict()}

    def next(self) -> Any:
        while True:
            item = next(self.node)
            r = self.rng.random()
            keep = r >= self.drop_below if self.drop_below is not None else r < self.p
            if keep != self.invert:
                return item


@register_transform("skip_random", SkipRandomConfig)
class SkipRandom(BaseTransform):
    def __init__(self, cfg, seed: int | None = None, **kwargs: Any):
        super().__init__(cfg)
        self.seed = seed                          # the pipeline's data seed; the config's own seed is added to it

    def build(self, source: BaseNode) -> BaseNode:
        seed = int(self.cfg.seed) if self.seed is None else int(self.seed) + int(self.cfg.seed)
        return SkipRandomNode(source, self.cfg, seed=seed)


# the reference's class names
SkipInterleavedTransform, SkipInterleavedTransformConfig, SkipInterleavedTransformNode = (
    SkipInterleaved, SkipInterleavedConfig, SkipInterleavedNode)
SkipRandomTransform, SkipRandomTransformConfig, SkipRandomTransformNode = SkipRandom, SkipRandomConfig, SkipRandomNode
