"""Sampling strategies for ``tokenized_dataset`` and their registry."""

from ....core.bootstrap import bootstrap_module
from ....core.registry import make_registry
from .base import BaseStrategy

_STRATEGY_REGISTRY, register_strategy, build_strategy = make_registry("dataset_sampling_strategy", BaseStrategy)
bootstrap_module(__name__)
