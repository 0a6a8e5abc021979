"""Serve recipe configuration (optimus_dl/recipe/serve/config.py:13-38)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

MISSING = "???"


@dataclass
class ServeCommonConfig:
    checkpoint_path: str | None = None   # load the model from a training checkpoint ...
    model: Any = None                    # ... or build it from a model config (exactly one of the two)
    tokenizer: Any = MISSING
    device: str = "auto"                 # cuda, cpu or auto
    dtype: str | None = None             # cast the served model (default: bf16 on CUDA, unchanged on CPU)
    use_kv_cache: bool = True
    seed: int = 0


@dataclass
class ServeRecipeConfig:
    port: int = 8000
    host: str = "0.0.0.0"


@dataclass
class ServeConfig:
    serve: ServeRecipeConfig = field(default_factory=ServeRecipeConfig)
    common: ServeCommonConfig = field(default_factory=ServeCommonConfig)
