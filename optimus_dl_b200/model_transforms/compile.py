"""``compile`` transform (optimus_dl/modules/model_transforms/compile.py:15-65).

The reference wraps the model in ``torch.compile``. Here the hot path is made of hand-written
kernels behind autograd functions, so tracing would add nothing and is not used: the transform
accepts the reference's config and returns the same model object. ``activation_memory_budget`` keeps its
meaning as far as it can without a compiler: the reference hands it to Inductor's partitioner, which recomputes
activations until only that fraction of them is kept (configs/train/train_llama_efficient.yaml uses 0.3); here a
budget ``b < 1`` turns on whole-block recomputation for ``round((1 - b) * n_blocks)`` evenly spaced transformer
blocks (the ``activation_checkpoint`` machinery), and a warning says so. ``use_inductor: true`` opts back into
``torch.compile`` for experiments on models that do not run the kernel path (CPU / fp32)."""

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
            budget = self.cfg.get("activation_memory_budget")
            if not kw.get("disable", False) and budget is not None and float(budget) < 1.0:
                self._recompute_blocks(model, float(budget))
            else:
                logger.info("compile transform: kernels are hand-written; model left as is")
            return model
        if self.cfg.activation_memory_budget is not None:
            import torch._functorch.config as fc

            fc.activation_memory_budget = float(self.cfg.activation_memory_budget)
        kw.pop("disable", None)
        return torch.compile(model, **kw)

    @staticmethod
    def _recompute_blocks(model: nn.Module, budget: float) -> None:
        from .checkpoint import checkpoint_module

        inner = getattr(model, "module", model)
        blocks = list(getattr(getattr(inner, "transformer", None), "h", []) or [])
        blocks = [b for b in blocks if not getattr(b, "_activation_checkpointed", False)]
        n = round((1.0 - max(budget, 0.0)) * len(blocks))
        if n <= 0 or not blocks:
            logger.warning("compile.activation_memory_budget=%.2f: no transformer blocks to recompute; nothing changed", budget)
            return
        picked = sorted({int(i * len(blocks) / n) for i in range(n)})
        for i in picked:
            checkpoint_module(blocks[i])
        logger.warning("compile.activation_memory_budget=%.2f is honoured by recomputing %d of %d transformer blocks "
                       "during backward (there is no compiler partitioner on this path)", budget, len(picked), len(blocks))
