"""Datasets and the ``dataset`` / ``dataset_sampling_strategy`` registries."""

from ...core.bootstrap import bootstrap_module
from ...core.registry import make_registry
from .base import BaseDataset

_DATASETS_REGISTRY, register_dataset, build_dataset = make_registry("dataset")
bootstrap_module(__name__)
