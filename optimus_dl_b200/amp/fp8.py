"""FP8 recipe surface (optimus_dl/modules/amp/fp8.py:40-523).

The reference drives NVIDIA Transformer Engine recipes; here FP8 means this package's own e4m3 GEMM
paths (``ops/fp8.py``). ``blockwise``: activations quantised per 1x128 block, weights per 128x128 block,
products scaled per 128-wide k-block. ``tensorwise``: one scale per tensor from its own maximum
(current scaling). ``delayed``: one scale per tensor from a history of maxima (``amax_history_len``,
``amax_compute_algo`` in {``max``, ``most_recent``}, ``margin``), refreshed once per backward pass.
``mxfp8`` is served by the ``blockwise`` implementation (the closest fine-grained scheme built here).
``FP8Recipe.autocast()`` switches the linear layers converted by the ``transformer_engine`` model
transform to the FP8 path for the duration of the context (forward and, through ``backward()``, the
backward pass). Enum names and string parsers follow the reference.
"""

from __future__ import annotations

import contextlib
import dataclasses
import enum
import logging
from typing import Any

import torch

from ..core.dtype import str_to_dtype

logger = logging.getLogger(__name__)


class Fp8Format(str, enum.Enum):
    HYBRID = "hybrid"
    E4M3 = "e4m3"
    E5M2 = "e5m2"


class Fp8RecipeType(str, enum.Enum):
    DELAYED = "delayed"
    TENSORWISE = "tensorwise"
    BLOCKWISE = "blockwise"
    MXFP8 = "mxfp8"


def parse_fp8_format(s: Any) -> Fp8Format:
    if isinstance(s, Fp8Format):
        return s
    key = str(s).strip().lower().replace("torch.", "")
    for affix in ("fp8_", "float8_"):
        key = key.removeprefix(affix)
    key = key.removesuffix("_fp8").removesuffix("fn")
    for f in Fp8Format:
        if key in (f.value, f.name.lower()):
            return f
    raise ValueError(f"Unknown FP8 format {s!r}; expected one of {[f.value for f in Fp8Format]}")


def parse_fp8_recipe(s: Any) -> Fp8RecipeType:
    if isinstance(s, Fp8RecipeType):
        return s
    key = str(s).strip().lower()
    aliases = {"current": "tensorwise", "block": "blockwise", "block_scaling": "blockwise", "mx": "mxfp8"}
    key = aliases.get(key, key)
    for r in Fp8RecipeType:
        if key == r.value:
            return r
    raise ValueError(f"unknown fp8 recipe {s!r}; expected one of {[r.value for r in Fp8RecipeType]}")


def get_fp8_format_from_string(format_str: str) -> Fp8Format:
    """Reference name of :func:`parse_fp8_format` (optimus_dl/modules/amp/fp8.py:96-119)."""
    return parse_fp8_format(format_str)


def get_fp8_recipe_type_from_string(recipe_str: str) -> Fp8RecipeType:
    """Reference name of :func:`parse_fp8_recipe` (optimus_dl/modules/amp/fp8.py:122-147)."""
    return parse_fp8_recipe(recipe_str)


def is_transformer_engine_available() -> bool:
    """Whether NVIDIA Transformer Engine can be imported. Nothing here depends on it: the FP8 path is this
    package's own kernels and works either way."""
    import importlib.util

    return importlib.util.find_spec("transformer_engine") is not None


def get_transformer_engine_version() -> str | None:
    if not is_transformer_engine_available():
        return None
    try:
        import transformer_engine

        return getattr(transformer_engine, "__version__", None)
    except Exception:
        return None


@dataclasses.dataclass
class Fp8RecipeConfig:
    """Arguments of :func:`create_fp8_recipe` as a dataclass (optimus_dl/modules/amp/fp8.py:150-178)."""

    recipe_type: str = "delayed"
    format: str = "hybrid"
    margin: int = 0
    amax_history_len: int = 1024
    amax_compute_algo: str = "max"
    reduce_amax: bool = True
    fp8_dpa: bool = False
    fp8_mha: bool = False


_state = {"enabled": False, "recipe": None}


def fp8_enabled() -> bool:
    """True inside an active ``FP8Recipe.autocast()`` context."""
    return bool(_state["enabled"])


class FP8Recipe:
    def __init__(self, fmt: Fp8Format = Fp8Format.E4M3, recipe: Fp8RecipeType = Fp8RecipeType.BLOCKWISE, **options: Any):
        self.format, self.recipe, self.options = fmt, recipe, options
        self.delayed_state = None
        if recipe == Fp8RecipeType.DELAYED:
            from ..ops.fp8 import DelayedScaling

            self.delayed_state = DelayedScaling(history=int(options.get("amax_history_len", 16) or 16),
                                                algo=str(options.get("amax_compute_algo", "max") or "max"),
                                                reduce_amax=bool(options.get("reduce_amax", True)))

    @contextlib.contextmanager
    def autocast(self, enabled: bool = True):
        prev = dict(_state)
        _state.update(enabled=enabled, recipe=self)
        try:
            yield self
        finally:
            _state.update(prev)

    @contextlib.contextmanager
    def backward(self, enabled: bool = True):
        """Context for the backward pass; on exit the delayed-scaling histories take this pass's maxima."""
        with self.autocast(enabled):
            yield self
        if enabled and self.delayed_state is not None:
            self.delayed_state.update(float(2.0 ** int(self.options.get("margin", 0) or 0)))

    def __repr__(self) -> str:
        return f"FP8Recipe(format={self.format.value}, recipe={self.recipe.value})"


def create_fp8_recipe(cfg: Any = None, format: Any = None, **kwargs: Any) -> FP8Recipe | None:
    """Recipe from an ``Fp8Config``-like mapping, or -- the reference's call form -- from
    ``(recipe_type, format, margin=..., amax_history_len=..., ...)`` / an :class:`Fp8RecipeConfig`.
    ``None`` when FP8 is off or no CUDA device exists."""
    if isinstance(cfg, Fp8RecipeConfig):
        cfg = dict(dataclasses.asdict(cfg), enabled=True)
        cfg["recipe"] = cfg.pop("recipe_type")
    elif isinstance(cfg, (str, Fp8RecipeType)) or (cfg is None and (format is not None or kwargs)):
        cfg = dict(kwargs, enabled=True, recipe=cfg if cfg is not None else kwargs.pop("recipe_type", "delayed"),
                   format=format if format is not None else "hybrid")
        cfg.pop("recipe_type", None)
    if cfg is None or not cfg.get("enabled", False):
        return None
    if not torch.cuda.is_available():
        logger.warning("fp8 requested but no CUDA device is present; running without fp8")
        return None
    fmt, rec = parse_fp8_format(cfg.get("format", "e4m3")), parse_fp8_recipe(cfg.get("recipe") or "delayed")
    if rec == Fp8RecipeType.MXFP8:
        logger.info("fp8 recipe mxfp8 is served by the block-scaled (1x128 / 128x128) e4m3 implementation")
    return FP8Recipe(fmt, rec, margin=cfg.get("margin", 0), amax_history_len=cfg.get("amax_history_len", 1024),
                     amax_compute_algo=cfg.get("amax_compute_algo", "max"), wgrad=bool(cfg.get("wgrad", True)),
                     reduce_amax=bool(cfg.get("reduce_amax", True)))


@contextlib.contextmanager
def fp8_autocast(device: torch.device, recipe: FP8Recipe | None, enabled: bool = True, dtype: Any = "bfloat16"):
    """FP8 context nested in bf16 autocast (or plain autocast when there is no recipe)."""
    dt = str_to_dtype(dtype) if dtype is not None else torch.bfloat16
    ac = torch.autocast(device_type=device.type, dtype=dt, enabled=enabled and device.type in ("cuda", "cpu"))
    if recipe is None:
        with ac:
            yield
    else:
        with ac, recipe.autocast(enabled):
            yield


def fp8_backward(recipe: FP8Recipe | None, enabled: bool = True):
    return recipe.backward(enabled) if recipe is not None else contextlib.nullcontext()
