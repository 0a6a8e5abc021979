"""``tensor_parallel`` transform (optimus_dl/modules/model_transforms/tensor_parallel.py:24-83).

Delegates to the model's ``apply_tp(tp_mesh, **custom_model_kwargs)``; skipped with a log line when
the collective has no tensor-parallel dimension (``tp_size == 1``) or is not mesh based.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any

import torch.nn as nn

from . import register_model_transform
from .base import BaseModelTransform
from .config import ModelTransformConfig

logger = logging.getLogger(__name__)


@dataclass
class TensorParallelConfig(ModelTransformConfig):
    custom_model_kwargs: dict = field(default_factory=dict)


@register_model_transform("tensor_parallel", TensorParallelConfig)
class TensorParallelTransform(BaseModelTransform):
    def apply(self, model: nn.Module, collective: Any = None, device: Any = None, **kwargs: Any) -> nn.Module:
        from ..parallel.collective import MeshCollective

        if not isinstance(collective, MeshCollective):
            logger.warning("tensor_parallel needs a mesh collective; transform skipped")
            return model
        if collective.tp_world_size <= 1:
            logger.info("no tensor-parallel mesh dimension (tp_size=1); transform skipped")
            return model
        if not hasattr(model, "apply_tp"):
            raise ValueError(f"{type(model).__name__} has no tensor-parallel plan (apply_tp)")
        extra = dict(self.cfg.custom_model_kwargs or {})
        if device is not None:
            extra.setdefault("device", device)
        model.apply_tp(collective.tp_mesh, **extra)
        logger.info("tensor parallelism applied over %d ranks (%s)", collective.tp_world_size, extra)
        return model
