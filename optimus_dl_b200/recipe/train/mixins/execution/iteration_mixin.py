"""One optimizer step (optimus_dl/recipe/train/mixins/execution/iteration_mixin.py:52-429):
micro-batch loop with gradient accumulation, loss scaling by ``1 / acc_steps``, gradient clipping,
scaler-aware optimizer step with ``pre/post_optimizer_step`` hooks and skipped-step detection,
timing and memory meters.

Timing: host wall-clock meters keep the reference's names (``perf/forward`` ...). Device time of the
whole step is measured with CUDA events and logged as ``perf/step_device_ms`` (read only on logging
steps, so no extra synchronisation otherwise).
"""

from __future__ import annotations

import logging
import time
from typing import Any, NamedTuple

import torch

from .....core.profile import get_sm_metrics, measured_next, nvtx_range
from .....metrics.base import meters_group
from .....metrics.common import log_averaged, log_summed
from .....model_transforms.distributed import accumulation_context
from .....parallel.fsdp import ShardedAdamW

logger = logging.getLogger(__name__)


class ForwardPassResult(NamedTuple):
    """Shape of one forward pass's outcome in the reference's step API
    (optimus_dl/recipe/train/mixins/execution/iteration_mixin.py:41-49); kept for code written against it."""

    loss: torch.Tensor
    exposed_protocols: dict[str, Any]
    elapsed_time: float


class OptimizerStepResult(NamedTuple):
    elapsed_time: float
    grad_norm: torch.Tensor | None


class TrainingIterationMixin:
    def log_memory_usage(self, device: torch.device) -> None:
        if device.type != "cuda":
            return
        log_averaged("gpu_gb_allocated", lambda: torch.cuda.memory_allocated(device) / 2**30, round=2)
        log_averaged("gpu_gb_used", lambda: torch.cuda.max_memory_allocated(device) / 2**30, round=2)
        log_averaged("gpu_gb_used_avg", lambda: torch.cuda.memory_reserved(device) / 2**30, round=2)
        sm = get_sm_metrics()
        if sm:
            for k, v in sm.items():
                log_averaged(k, v, round=1)

    def run_training_iteration(self, model: torch.nn.Module, optimizer: Any, criterion: Any, train_data_iter: Any,
                               training_context: dict[str, Any], lr_scheduler: Any = None, acc_steps: int = 1,
                               clip_grad_norm: float | None = None, log_freq: int | None = None,
                               metric_engine: Any = None, collective: Any = None) -> bool:
        device = training_context["device"]
        scaler = training_context["scaler"]
        if scaler is not None and not scaler.is_enabled():
            scaler = None                      # a disabled scaler scales nothing: take the plain path
        with meters_group("train", log_freq=log_freq) as should_log:
            optimizer.zero_grad()
            model.train()
            ev0 = ev1 = None
            if should_log and device.type == "cuda":
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            t_get = t_fwd = t_bwd = 0.0
            if hasattr(criterion, "grad_scale"):
                criterion.grad_scale = 1.0 / acc_steps
            requested = metric_engine.required_external_protocols if (metric_engine is not None and should_log) else None
            for mb in range(acc_steps):
                ms, batch = measured_next(train_data_iter)
                t_get += ms
                last = mb == acc_steps - 1
                with accumulation_context(model, last):
                    t0 = time.perf_counter()
                    with training_context["amp_ctx"](), nvtx_range("train/forward"):
                        loss, exposed = criterion(model, batch, requested_protocols=requested)
                    loss = loss / acc_steps
                    t_fwd += (time.perf_counter() - t0) * 1e3
                    if metric_engine is not None and should_log:
                        metric_engine.update(dict(model=model, batch=batch), exposed)
                    t0 = time.perf_counter()
                    with training_context["fp8_backward_ctx"](), nvtx_range("train/backward"):
                        (scaler.scale(loss) if scaler is not None else loss).backward()
                    t_bwd += (time.perf_counter() - t0) * 1e3
            log_averaged("perf/batch_get", t_get, round=2)
            log_averaged("perf/forward", t_fwd, round=2)
            log_averaged("perf/backward", t_bwd, round=2)
            t0 = time.perf_counter()
            with nvtx_range("train/optimizer"):
                skipped = self._optimizer_step(model, optimizer, scaler, clip_grad_norm)
            log_averaged("perf/optimizer", (time.perf_counter() - t0) * 1e3, round=2)
            if ev1 is not None:
                ev1.record()
                log_averaged("perf/step_device_ms", lambda: (ev1.synchronize(), ev0.elapsed_time(ev1))[1], round=2)
            log_averaged("learning_rate", lambda: optimizer.param_groups[0]["lr"])
            log_summed("optimizer_step_skipped", float(skipped))
            if scaler is not None:
                log_averaged("grad_scale", lambda: scaler.get_scale())
            self.log_memory_usage(device)
            optimizer.zero_grad()
            if lr_scheduler is not None:
                lr_scheduler.step()
        return should_log

    def _optimizer_step(self, model: torch.nn.Module, optimizer: Any, scaler: Any, clip: float | None) -> bool:
        sharded = isinstance(optimizer, ShardedAdamW)
        if scaler is not None:
            scaler.unscale_(optimizer)
        if clip and not sharded:
            norm = torch.nn.utils.clip_grad_norm_([p for g in optimizer.param_groups for p in g["params"]], float(clip))
            log_averaged("grad_norm", lambda: norm.item(), round=4)
        if hasattr(model, "pre_optimizer_step"):
            model.pre_optimizer_step()
        skipped = False
        if scaler is not None:
            before = scaler.get_scale()
            scaler.step(optimizer)
            scaler.update()
            skipped = scaler.get_scale() < before
        else:
            optimizer.step()
        if sharded and clip:
            log_averaged("grad_norm", lambda: optimizer.grad_norm().item(), round=4)
        if hasattr(model, "post_optimizer_step"):
            model.post_optimizer_step()
        return skipped
