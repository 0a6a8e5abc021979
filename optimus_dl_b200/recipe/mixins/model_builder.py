"""Model builder (optimus_dl/recipe/mixins/model_builder.py:27-120): build from the ``model`` registry,
log parameter counts, apply the configured transforms in order. Each transform receives
``collective``, ``device``, ``is_restart`` and ``checkpoint_manager``.

On a CUDA device the model is constructed directly on the device in bf16 when the first
transform is ``fully_shard`` (fp32 masters are taken by the sharding engine), which avoids a full
fp32 host copy of multi-billion-parameter models."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

import torch

from ...core.model_utils import get_num_parameters
from ...core.registry import RegistryConfig, make_registry
from ...metrics.common import log_averaged, log_summed
from ...model_transforms import build_model_transform
from ...models import build_model

logger = logging.getLogger(__name__)


@dataclass
class ModelBuilderConfig(RegistryConfig):
    pass


class ModelBuilder:
    def __init__(self, cfg: Any = None, model_transforms: Any = None, **kwargs: Any):
        self.cfg = cfg
        self.model_transforms = list(model_transforms or [])

    def build_model(self, model_config: Any, collective: Any = None, device: Any = None, is_restart: bool = False,
                    checkpoint_manager: Any = None, **kwargs: Any) -> torch.nn.Module:
        names = [t.get("_name") if hasattr(t, "get") else None for t in self.model_transforms]
        on_device = device is not None and getattr(device, "type", None) == "cuda" and "fully_shard" in names
        if on_device:
            prev = torch.get_default_dtype()
            torch.set_default_dtype(torch.bfloat16)
            try:
                with torch.device(device):
                    model = build_model(model_config, **kwargs)
            finally:
                torch.set_default_dtype(prev)
        else:
            model = build_model(model_config, **kwargs)
        n_all, n_train = get_num_parameters(model), get_num_parameters(model, only_trainable=True)
        logger.info("model has %.2fM parameters (%.2fM trainable)", n_all / 1e6, n_train / 1e6)
        log_summed("model/num_params_total", n_all, reset=False)
        log_summed("model/num_params_trainable", n_train, reset=False)
        # the two meters of optimus_dl/recipe/mixins/model_builder.py:74-86 (averaged over ranks)
        log_averaged("model/num_params_before_transforms", n_all)
        model = self.apply_transforms(model, collective=collective, device=device, is_restart=is_restart,
                                      checkpoint_manager=checkpoint_manager)
        log_averaged("model/num_params_after_transforms", lambda: get_num_parameters(model))
        return model

    def apply_transforms(self, model: torch.nn.Module, **kwargs: Any) -> torch.nn.Module:
        for tcfg in self.model_transforms:
            if hasattr(tcfg, "get") and tcfg.get("enabled", True) is False:
                continue
            transform = build_model_transform(tcfg)
            logger.info("applying model transform %s", tcfg.get("_name") if hasattr(tcfg, "get") else tcfg)
            model = transform.apply(model, **kwargs)
        return model


_MB_REGISTRY, register_model_builder, build_model_builder = make_registry("model_builder")
register_model_builder("base", ModelBuilderConfig)(ModelBuilder)
