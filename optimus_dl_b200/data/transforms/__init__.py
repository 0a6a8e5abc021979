"""Pipeline transforms and the ``transform`` registry."""

from ...core.bootstrap import bootstrap_module
from ...core.registry import make_registry
from .base import BaseTransform

_TRANSFORMS_REGISTRY, register_transform, build_transform = make_registry("transform", BaseTransform)
bootstrap_module(__name__)
