"""Transform interface (optimus_dl/modules/model_transforms/base.py:13-48)."""

from __future__ import annotations

from typing import Any

import torch.nn as nn


class BaseModelTransform:
    def __init__(self, cfg: Any = None, **kwargs: Any):
        self.cfg = cfg

    def apply(self, model: nn.Module, **kwargs: Any) -> nn.Module:
        """Return the transformed model. ``kwargs`` carry ``collective``, ``device``, ``is_restart``,
        ``checkpoint_manager`` from the model builder."""
        raise NotImplementedError
