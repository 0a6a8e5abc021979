"""``ddp`` and ``fully_shard`` transforms (optimus_dl/modules/model_transforms/distributed.py:48-332).

``fully_shard`` hands the model to this package's sharding engine (``parallel/fsdp.py``): one group
per transformer block plus a root group, bf16 compute parameters, fp32 master shards, gradient
averaging over the data-parallel ranks. The reference's knobs:
``reshard_after_forward`` (``true`` or a positive int: a block's gathered parameters live in a small
pool of buffers and are gathered again for its backward; together with the model's
``shard_every_ith_layer`` only every i-th block does so), ``mixed_precision`` (``param_dtype`` must be
bf16 and ``reduce_dtype`` fp32, which is what the reduce kernel does; ``output_dtype`` is refused, the
blocks return bf16), ``offload`` (``cpu_offload: true`` is refused: optimizer state lives sharded in
HBM), ``sync_grad_accum`` (gradients are reduced after every micro-batch in either setting: no rank
keeps full-size gradients) and ``use_hybrid_sharding`` (the shard group is the ``dp_shard`` mesh
dimension; replicas across ``dp_replicate`` are averaged with NCCL after the in-kernel reduce).
``accumulation_context(model, is_last)`` tells the engine which micro-batch ends the step.
"""

from __future__ import annotations

import contextlib
import logging
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn as nn

from ..core.registry import RegistryConfig
from ..models.base import BaseModel
from . import register_model_transform
from .base import BaseModelTransform

logger = logging.getLogger(__name__)


@dataclass
class DDPTransformConfig(RegistryConfig):
    find_unused_parameters: bool = False
    gradient_as_bucket_view: bool = True
    static_graph: bool = False
    broadcast_buffers: bool = True


class DDPWrappedModel(nn.parallel.DistributedDataParallel):
    """DDP that still exposes the BaseModel hooks of the wrapped model."""

    def make_parameter_groups(self):
        return self.module.make_parameter_groups()

    def accumulation_context(self, is_last_microbatch: bool):
        return contextlib.nullcontext() if is_last_microbatch else self.no_sync()

    def __getattr__(self, name: str):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)


@register_model_transform("ddp", DDPTransformConfig)
class DDPTransform(BaseModelTransform):
    def apply(self, model: nn.Module, collective: Any = None, device: Any = None, **kwargs: Any) -> nn.Module:
        if collective is None or collective.world_size == 1:
            logger.warning("ddp transform: single process, model left unwrapped")
            return model.to(device) if device is not None else model
        if getattr(collective, "shard_world_size", 1) != 1:
            raise ValueError("ddp needs sharding_world_size == 1 (every data-parallel rank holds full parameters)")
        model = model.to(device)
        ids = [device.index] if device is not None and device.type == "cuda" else None
        return DDPWrappedModel(model, device_ids=ids, process_group=collective.process_group,
                               find_unused_parameters=bool(self.cfg.find_unused_parameters),
                               gradient_as_bucket_view=bool(self.cfg.gradient_as_bucket_view),
                               static_graph=bool(self.cfg.static_graph),
                               broadcast_buffers=bool(self.cfg.broadcast_buffers))


@dataclass
class MixedPrecisionConfig:
    param_dtype: str | None = "bfloat16"
    reduce_dtype: str | None = "float32"
    output_dtype: str | None = None
    cast_forward_inputs: bool = True
    fp8_enabled: bool = False        # informational, as in the reference: FP8 is driven by optimization.amp.fp8
    fp8_format: str | None = None


@dataclass
class OffloadConfig:
    """CPU offload policy of the reference's config tree (optimus_dl/modules/model_transforms/distributed.py:172-182).
    ``cpu_offload: true`` is refused: parameters and optimizer state live sharded in HBM here."""

    cpu_offload: bool = False
    pin_memory: bool = True


def _wants_cpu_offload(value: Any) -> bool:
    """``offload`` may be a bool (this package's short form) or the reference's nested ``{cpu_offload, pin_memory}``."""
    if value is None or isinstance(value, bool):
        return bool(value)
    getter = value.get if hasattr(value, "get") else (lambda k, d=None: getattr(value, k, d))
    return bool(getter("cpu_offload", False))


@dataclass
class FullyShardTransformConfig(RegistryConfig):
    reshard_after_forward: Any = False
    mixed_precision: MixedPrecisionConfig | None = None
    offload: Any = None
    pin_memory: bool = True
    sync_grad_accum: bool = False
    use_hybrid_sharding: bool = True
    fuse_optimizer_in_backward: bool = True
    copy_ctas: int = 16
    pull_ctas: int = 24
    param_slots: int = 2         # pool size for resharded blocks (reshard_after_forward)


@register_model_transform("fully_shard", FullyShardTransformConfig)
class FullyShardTransform(BaseModelTransform):
    def apply(self, model: nn.Module, collective: Any = None, device: Any = None, **kwargs: Any) -> nn.Module:
        from ..parallel.fsdp import FSDPConfig, fully_shard_model

        if _wants_cpu_offload(self.cfg.offload):
            raise ValueError("fully_shard: CPU offload is not supported; optimizer state is sharded in HBM")
        mp = self.cfg.get("mixed_precision")
        if mp is not None and mp.get("param_dtype") not in (None, "bfloat16", "bf16", "torch.bfloat16"):
            raise ValueError("fully_shard: compute parameters are bf16 on this engine")
        if mp is not None and mp.get("reduce_dtype") not in (None, "float32", "fp32", "torch.float32"):
            raise ValueError("fully_shard: gradients are reduced and accumulated in fp32 on this engine "
                             f"(mixed_precision.reduce_dtype={mp.get('reduce_dtype')!r} is not available)")
        if mp is not None and mp.get("output_dtype") not in (None, "bfloat16", "bf16", "torch.bfloat16"):
            raise ValueError("fully_shard: block outputs are bf16 on this engine (mixed_precision.output_dtype)")
        if mp is not None and mp.get("cast_forward_inputs", True) is False:
            logger.warning("fully_shard: cast_forward_inputs=false has no effect (token ids are the only model inputs)")
        device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        if device.type != "cuda":
            logger.warning("fully_shard: no CUDA device; model left unsharded (fp32, single process semantics)")
            return model.to(device)
        group = rep_group = None
        rep_world = 1
        if collective is not None and collective.world_size > 1:
            mesh = getattr(collective, "parallel_mesh", None)
            group = mesh.get_group("dp_shard") if mesh is not None else collective.process_group
            if mesh is not None and mesh["dp_replicate"].size() > 1:
                if bool(self.cfg.use_hybrid_sharding):
                    # shard inside dp_shard (NVLink domain), sum gradients over dp_replicate
                    rep_group, rep_world = mesh.get_group("dp_replicate"), mesh["dp_replicate"].size()
                else:
                    # one flat shard group over every data-parallel rank
                    group = mesh["dp_replicate", "dp_shard"]._flatten("dp").get_group()
        raf = self.cfg.reshard_after_forward
        if isinstance(raf, int) and not isinstance(raf, bool) and raf > 1:
            logger.warning("fully_shard: reshard_after_forward=%d (reshard to a smaller group) is treated as true: "
                           "gathered parameters are freed completely after use", raf)
        cfg = FSDPConfig(reshard_after_forward=bool(raf), param_slots=int(self.cfg.get("param_slots", 2) or 2),
                         fuse_optimizer_in_backward=bool(self.cfg.fuse_optimizer_in_backward),
                         copy_ctas=int(self.cfg.copy_ctas), pull_ctas=int(self.cfg.pull_ctas),
                         sync_grad_accum=bool(self.cfg.sync_grad_accum))
        engine = fully_shard_model(model, group, device, cfg)
        engine.replicate_group, engine.replicate_world = rep_group, rep_world
        return model


BaseDistributedTransform = BaseModelTransform   # the reference's name for the common base of ddp / fully_shard


def accumulation_context(model: nn.Module, is_last_microbatch: bool):
    """Context for one micro-batch: gradient synchronisation only happens on the last one."""
    if hasattr(model, "accumulation_context"):
        return model.accumulation_context(is_last_microbatch)
    eng = getattr(model, "_sharding_engine", None)
    if eng is None:
        return contextlib.nullcontext()

    @contextlib.contextmanager
    def ctx():
        eng.set_requires_gradient_sync(is_last_microbatch)
        try:
            yield
        finally:
            eng.set_requires_gradient_sync(True)

    return ctx()
