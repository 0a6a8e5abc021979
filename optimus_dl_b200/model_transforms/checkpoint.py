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


class CheckpointWrapper(nn.Module):
    """Marker base of checkpointed modules (class name of optimus_dl/modules/model_transforms/checkpoint.py:24-60).

    A module is checkpointed by giving it a subclass of its own class that also derives from this one, under the same
    class name: ``isinstance(m, CheckpointWrapper)`` holds, ``m.module`` is the module itself, and neither parameter
    names nor class-name matching by later transforms change."""

    _ckpt_ctx_fn: Any = None
    use_reentrant: bool = False

    @property
    def module(self) -> nn.Module:
        return self

    def forward(self, *args: Any, **kwargs: Any):
        inner = self.__dict__.get("_ckpt_inner_forward") or super().forward
        if not torch.is_grad_enabled():
            return inner(*args, **kwargs)
        extra = {"context_fn": self._ckpt_ctx_fn} if self._ckpt_ctx_fn is not None else {}
        return checkpoint(inner, *args, use_reentrant=self.use_reentrant, **extra, **kwargs)


@functools.lru_cache(maxsize=None)
def _checkpointed_class(cls: type) -> type:
    return type(cls.__name__, (CheckpointWrapper, cls), {"__module__": cls.__module__, "__qualname__": cls.__qualname__})


def checkpoint_module(m: nn.Module, ctx_fn: Any = None, use_reentrant: bool = False) -> None:
    """Make ``m`` recompute its forward during backward, in place: hooks registered on the module keep firing once
    per outer call and not during the recomputation."""
    if not isinstance(m, CheckpointWrapper):
        m.__class__ = _checkpointed_class(type(m))
    if "forward" in m.__dict__:          # a forward set on the instance would hide the class's: it becomes the inner one
        m._ckpt_inner_forward = m.__dict__.pop("forward")
    m._ckpt_ctx_fn = ctx_fn
    m.use_reentrant = bool(use_reentrant)
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
