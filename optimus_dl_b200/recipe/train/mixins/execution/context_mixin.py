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


class FreshContext:
    """A context factory that is also a context manager: ``with ctx:`` (how the reference's training loop uses the
    entries of the training context) and ``with ctx():`` both enter a NEW context from ``factory``, so the object
    can be entered any number of times, nested included."""

    def __init__(self, factory: Any):
        self._factory = factory
        self._open: list[Any] = []

    def __call__(self) -> Any:
        return self._factory()

    def __enter__(self) -> Any:
        ctx = self._factory()
        self._open.append(ctx)
        return ctx.__enter__()

    def __exit__(self, *exc: Any) -> Any:
        return self._open.pop().__exit__(*exc)


class TrainingContextMixin:
    def __init__(self, optimization_config: Any = None, **kwargs: Any):
        self.optimization_config = optimization_config
        self._fp8_recipe = None

    def get_fp8_backward_ctx(self) -> Any:
        """Context for the backward pass: the FP8 recipe's when one is active, else a null context."""
        recipe = getattr(self, "_fp8_recipe", None)
        return fp8_backward(recipe) if recipe is not None else contextlib.nullcontext()

    def setup_training_context(self, device: torch.device, amp_cfg: Any = None) -> dict[str, Any]:
        """``scaler`` (always a ``torch.GradScaler``; enabled only for fp16-style AMP on CUDA, never with FP8),
        ``amp_ctx`` / ``fp8_backward_ctx`` (:class:`FreshContext`), ``amp_cfg``, ``device``, ``fp8_recipe``,
        ``fp8_enabled``, ``is_fp8_dtype``. FP8 is on when AMP is enabled, the dtype is an fp8 type AND ``fp8.enabled``
        is set (the rule of optimus_dl/recipe/train/mixins/execution/context_mixin.py:69-99); an fp8 dtype without
        ``fp8.enabled`` falls back to bf16 autocast."""
        if amp_cfg is None:
            opt = getattr(self, "optimization_config", None)
            amp_cfg = (opt.get("amp") if hasattr(opt, "get") else getattr(opt, "amp", None)) if opt is not None else None
        get = (lambda k, d=None: amp_cfg.get(k, d) if hasattr(amp_cfg, "get") else getattr(amp_cfg, k, d)) \
            if amp_cfg is not None else (lambda k, d=None: d)
        enabled = bool(get("enabled", False))
        dtype_name = get("dtype", "bfloat16") or "bfloat16"
        fp8_dtype = is_fp8_dtype(dtype_name)
        fp8_cfg = get("fp8")
        fp8_get = (lambda k, d=None: fp8_cfg.get(k, d) if hasattr(fp8_cfg, "get") else getattr(fp8_cfg, k, d)) \
            if fp8_cfg is not None else (lambda k, d=None: d)
        fp8_wanted = bool(fp8_get("enabled", False))
        fp8_recipe = None
        if enabled and fp8_dtype and fp8_wanted:
            if hasattr(fp8_cfg, "items"):
                cfg = dict(fp8_cfg)
            else:
                import dataclasses

                cfg = dataclasses.asdict(fp8_cfg)
            cfg["enabled"] = True
            cfg.setdefault("format", "e4m3" if "e4m3" in str(dtype_name) or str(dtype_name) == "fp8" else "e5m2")
            fp8_recipe = create_fp8_recipe(cfg)
        elif enabled and (fp8_dtype or fp8_wanted):
            logger.warning("FP8 needs both an fp8 amp.dtype and amp.fp8.enabled (dtype=%s, fp8.enabled=%s): "
                           "running bf16 autocast", dtype_name, fp8_wanted)
        self._fp8_recipe = fp8_recipe
        compute_dtype = torch.bfloat16 if fp8_dtype else str_to_dtype(dtype_name)
        use_scaler = enabled and bool(get("enable_scaler", False)) and not fp8_dtype and device.type == "cuda"
        scaler = torch.GradScaler(device="cuda" if device.type == "cuda" else "cpu", enabled=use_scaler,
                                  init_scale=float(get("init_scale", 65536.0)),
                                  growth_factor=float(get("growth_factor", 2.0)),
                                  backoff_factor=float(get("backoff_factor", 0.5)),
                                  growth_interval=int(get("growth_interval", 2000)))

        def amp_ctx():
            if not enabled:
                return contextlib.nullcontext()
            if fp8_recipe is not None:
                return fp8_autocast(device, fp8_recipe, True, compute_dtype)
            if device.type in ("cuda", "cpu"):
                return torch.autocast(device_type=device.type, dtype=compute_dtype)
            return contextlib.nullcontext()

        return {"scaler": scaler, "amp_ctx": FreshContext(amp_ctx), "amp_cfg": amp_cfg, "device": device,
                "fp8_recipe": fp8_recipe, "fp8_enabled": fp8_recipe is not None, "is_fp8_dtype": fp8_dtype,
                "fp8_backward_ctx": FreshContext(self.get_fp8_backward_ctx)}
