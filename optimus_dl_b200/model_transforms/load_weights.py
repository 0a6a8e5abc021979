"""``load_weights`` transform (optimus_dl/modules/model_transforms/load_weights.py:18-77): initialise
the model from another checkpoint (a DCP directory, an output directory or a ``.pt`` file); skipped
on restart when ``skip_on_restart`` is set, because the run's own checkpoint wins."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

import torch.nn as nn

from ..core.registry import RegistryConfig
from . import register_model_transform
from .base import BaseModelTransform

logger = logging.getLogger(__name__)


@dataclass
class LoadWeightsConfig(RegistryConfig):
    path: str | None = None
    checkpoint_path: str | None = None   # the reference's name for ``path``
    strict: bool = True
    skip_on_restart: bool = True


@register_model_transform("load_weights", LoadWeightsConfig)
class LoadWeightsTransform(BaseModelTransform):
    def apply(self, model: nn.Module, is_restart: bool = False, checkpoint_manager: Any = None, **kwargs: Any) -> nn.Module:
        if is_restart and self.cfg.skip_on_restart:
            logger.info("load_weights: restart detected, keeping the run's own checkpoint")
            return model
        from ..checkpoint import CheckpointManager

        mgr = checkpoint_manager or CheckpointManager()
        path = self.cfg.checkpoint_path if self.cfg.checkpoint_path is not None else self.cfg.path
        if path is None:
            raise ValueError("load_weights: set checkpoint_path (or path)")
        path = str(path)
        cp = mgr.get_checkpoint(path)
        mgr.load_model_state_dict(model, cp.checkpoint if cp is not None else path, strict=bool(self.cfg.strict))
        logger.info("loaded weights from %s", path)
        return model


LoadWeightsTransformConfig = LoadWeightsConfig   # the reference's name
