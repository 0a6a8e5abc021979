"""Datasets and the ``dataset`` / ``dataset_sampling_strategy`` registries."""

from ...core.bootstrap import bootstrap_module
from ...core.registry import make_registry
from .base import BaseDataset

_DATASETS_REGISTRY, register_dataset, build_dataset = make_registry("dataset")
bootstrap_module(__name__)
from .. import presets as _presets  # noqa: E402,F401  (registers preset_* datasets)
from ..presets import corpora as _corpora  # noqa: E402,F401
