"""``prefetch``: run the upstream pipeline on a background thread
(optimus_dl/modules/data/transforms/prefetch.py)."""

from __future__ import annotations

from dataclasses import dataclass

from torchdata.nodes import BaseNode, Prefetcher

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform


@dataclass
class PrefetchTransformConfig(RegistryConfigStrict):
    prefetch_factor: int = 8
    snapshot_frequency: int = 128


@register_transform("prefetch", PrefetchTransformConfig)
class PrefetchTransform(BaseTransform):
    def build(self, source: BaseNode) -> BaseNode:
        return Prefetcher(source, prefetch_factor=int(self.cfg.prefetch_factor),
                          snapshot_frequency=int(self.cfg.snapshot_frequency))
