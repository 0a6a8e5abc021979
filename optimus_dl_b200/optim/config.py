"""Optimization, AMP and FP8 configs (optimus_dl/modules/optim/config.py:16-130)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class Fp8Config:
    """FP8 settings. ``recipe: blockwise`` selects the block-scaled e4m3 GEMMs (1x128 activation scales,
    128x128 weight scales); ``tensorwise`` / ``delayed`` select per-tensor scales (``margin``,
    ``amax_history_len``, ``amax_compute_algo`` apply to ``delayed``; ``wgrad`` chooses FP8 or bf16 weight
    gradients for both). Fields the reference declares but never reads (``param``,
    ``first_last_layers_bf16``, ``tp_only_amax_red``) are accepted."""

    enabled: bool = False
    format: str = "hybrid"            # hybrid | e4m3 | e5m2
    recipe: str = "delayed"           # delayed | tensorwise | blockwise | mxfp8
    param: bool = False
    margin: int = 0
    amax_history_len: int = 1024
    amax_compute_algo: str = "max"
    reduce_amax: bool = True
    wgrad: bool = True
    fp8_dpa: bool = False
    fp8_mha: bool = False
    first_last_layers_bf16: bool = False
    num_layers_at_start_in_bf16: int = 1
    num_layers_at_end_in_bf16: int = 1
    tp_only_amax_red: bool = False


@dataclass
class AmpConfig:
    enabled: bool = False
    dtype: str = "bfloat16"
    enable_scaler: Any = "${eval:'\"${.dtype}\" in (\"float16\", \"fp16\", \"half\", \"torch.float16\", \"torch.half\")'}"
    init_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    fp8: Fp8Config = field(default_factory=Fp8Config)


@dataclass
class OptimizationConfig:
    optimizer: Any = "???"
    iterations: int = 1000
    acc_steps: int = 1
    clip_grad_norm: float | None = None
    amp: AmpConfig = field(default_factory=AmpConfig)
