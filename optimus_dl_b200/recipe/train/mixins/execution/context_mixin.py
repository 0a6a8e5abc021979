"""Training context (optimus_dl/recipe/train/mixins/execution/context_mixin.py:29-181): grad scaler,
autocast context (bf16 / fp16, or the FP8 recipe nested in bf16 autocast) and related flags."""

from __future__ import annotations

import contextlib
import logging
from typing import Any

import torch

from .....amp.fp8 import create_fp8_recipe, fp8_autocast, fp8_backward
from .....core.dtype import is_fp8_dtype, str_to_dtype

logger = logging.getLogger(__name__)


class TrainingContextMixin:
    def setup_training_context(self, device: torch.device, amp_cfg: Any = None) -> dict[str, Any]:
        amp_cfg = amp_cfg if amp_cfg is not None else getattr(self, "optimization_config", {}).get("amp")
        enabled = bool(amp_cfg.get("enabled", False)) if amp_cfg is not None else False
        dtype_name = amp_cfg.get("dtype", "bfloat16") if amp_cfg is not None else "bfloat16"
        fp8_dtype = is_fp8_dtype(dtype_name)
        fp8_cfg = amp_cfg.get("fp8") if amp_cfg is not None else None
        fp8_recipe = None
        if enabled and (fp8_dtype or (fp8_cfg is not None and fp8_cfg.get("enabled", False))):
            cfg = dict(fp8_cfg or {})
            cfg["enabled"] = True
            if fp8_dtype:
                cfg.setdefault("format", "e4m3" if "e4m3" in str(dtype_name) or str(dtype_name) == "fp8" else "e5m2")
            fp8_recipe = create_fp8_recipe(cfg)
        compute_dtype = torch.bfloat16 if fp8_dtype else str_to_dtype(dtype_name)
        use_scaler = bool(amp_cfg.get("enable_scaler", False)) if (enabled and amp_cfg is not None) else False
        scaler = None
        if use_scaler and device.type == "cuda":
            scaler = torch.amp.GradScaler("cuda", init_scale=float(amp_cfg.get("init_scale", 65536.0)),
                                          growth_factor=float(amp_cfg.get("growth_factor", 2.0)),
                                          backoff_factor=float(amp_cfg.get("backoff_factor", 0.5)),
                                          growth_interval=int(amp_cfg.get("growth_interval", 2000)))

        def amp_ctx():
            if not enabled:
                return contextlib.nullcontext()
            if fp8_recipe is not None:
                return fp8_autocast(device, fp8_recipe, True, compute_dtype)
            if device.type in ("cuda", "cpu"):
                return torch.autocast(device_type=device.type, dtype=compute_dtype)
            return contextlib.nullcontext()

        return {"scaler": scaler, "amp_ctx": amp_ctx, "amp_cfg": amp_cfg, "device": device, "fp8_recipe": fp8_recipe,
                "fp8_enabled": fp8_recipe is not None, "is_fp8_dtype": fp8_dtype,
                "fp8_backward_ctx": (lambda: fp8_backward(fp8_recipe))}
