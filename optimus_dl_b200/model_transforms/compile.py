"""``compile`` transform (optimus_dl/modules/model_transforms/compile.py:15-65).

The reference wraps the model in ``torch.compile``. Here the hot path is made of hand-written
kernels behind autograd functions, so tracing would add nothing and is not used: the transform
accepts the reference's config (``compile_kwargs``, ``activation_memory_budget``) and returns the model
unchanged. ``use_inductor: true`` opts back into ``torch.compile`` for experiments on models that do
not run the kernel path (CPU / fp32)."""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn as nn

from ..core.registry import RegistryConfig
from . import register_model_transform
from .base import BaseModelTransform

logger = logging.getLogger(__name__)


@dataclass
class CompileTransformConfig(RegistryConfig):
    compile_kwargs: dict = field(default_factory=dict)
    activation_memory_budget: float | None = 1.0
    use_inductor: bool = False
    enabled: bool = True


@register_model_transform("compile", CompileTransformConfig)
class CompileTransform(BaseModelTransform):
    def apply(self, model: nn.Module, **kwargs: Any) -> nn.Module:
        kw = dict(self.cfg.get("compile_kwargs") or {})
        if kw.get("disable", False) or not self.cfg.get("use_inductor", False):
            logger.info("compile transform: kernels are hand-written; model left as is")
            return model
        if self.cfg.activation_memory_budget is not None:
            import torch._functorch.config as fc

            fc.activation_memory_budget = float(self.cfg.activation_memory_budget)
        kw.pop("disable", None)
        return torch.compile(model, **kw)
