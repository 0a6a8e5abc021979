"""``activation_checkpoint`` transform (optimus_dl/modules/model_transforms/checkpoint.py:24-158).

Modules whose class name is listed in ``layer_classes`` recompute their forward during backward
(non-reentrant ``torch.utils.checkpoint``), optionally with a selective policy: ops named in
``ops_to_save`` keep their outputs, everything else is recomputed. Unlike the reference, the wrapped
module keeps its place in the tree (its ``forward`` is replaced), so state-dict keys do not gain a
``.module.`` segment."""

from __future__ import annotations

import functools
import logging
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn as nn
from torch.utils.checkpoint import CheckpointPolicy, checkpoint, create_selective_checkpoint_contexts

from ..core.conf import locate
from ..core.registry import RegistryConfig
from . import register_model_transform
from .base import BaseModelTransform

logger = logging.getLogger(__name__)


@dataclass
class ActivationCheckpointConfig(RegistryConfig):
    layer_classes: list[str] = field(default_factory=list)
    ops_to_save: list[str] = field(default_factory=list)
    every_nth: int = 1
    use_reentrant: bool = False


def _policy(ops: list[Any]):
    saved = set(ops)

    def policy(ctx, op, *args, **kwargs):
        return CheckpointPolicy.MUST_SAVE if op in saved else CheckpointPolicy.PREFER_RECOMPUTE

    return policy


def checkpoint_module(m: nn.Module, ctx_fn: Any = None, use_reentrant: bool = False) -> None:
    """Make ``m`` recompute its forward during backward (its ``forward`` is wrapped in place, so hooks registered on
    the module keep firing once per outer call and not during the recomputation)."""
    orig = m.forward

    def wrapped(*a, _orig=orig, **k):
        if not torch.is_grad_enabled():
            return _orig(*a, **k)
        extra = {"context_fn": ctx_fn} if ctx_fn is not None else {}
        return checkpoint(_orig, *a, use_reentrant=use_reentrant, **extra, **k)

    m.forward = wrapped
    m._activation_checkpointed = True


@register_model_transform("activation_checkpoint", ActivationCheckpointConfig)
class ActivationCheckpointTransform(BaseModelTransform):
    def apply(self, model: nn.Module, **kwargs: Any) -> nn.Module:
        names = set(self.cfg.layer_classes or [])
        ops = []
        for o in (self.cfg.ops_to_save or []):
            try:
                ops.append(locate(o) if isinstance(o, str) else o)
            except Exception:
                logger.warning("activation_checkpoint: cannot resolve op %r", o)
        ctx_fn = functools.partial(create_selective_checkpoint_contexts, _policy(ops)) if ops else None
        count = 0
        for i, m in enumerate([m for m in model.modules() if type(m).__name__ in names]):
            if i % max(1, int(self.cfg.every_nth)) != 0:
                continue
            checkpoint_module(m, ctx_fn, bool(self.cfg.get("use_reentrant", False)))
            count += 1
        logger.info("activation checkpointing enabled on %d modules", count)
        return model
