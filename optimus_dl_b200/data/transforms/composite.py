"""``compose``: apply transforms in order (optimus_dl/modules/data/transforms/composite.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfig
from . import build_transform, register_transform
from .base import BaseTransform


@dataclass
class CompositeTransformConfig(RegistryConfig):
    transforms: list[Any] = field(default_factory=list)


@register_transform("compose", CompositeTransformConfig)
class CompositeTransform(BaseTransform):
    def __init__(self, cfg, **kwargs: Any):
        super().__init__(cfg)
        self.transforms = [build_transform(t, **kwargs) for t in (cfg.transforms or [])]

    def build(self, source: BaseNode) -> BaseNode:
        node = source
        for t in self.transforms:
            node = t.build(node)
        return node
