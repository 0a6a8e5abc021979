"""String -> ``torch.dtype`` parsing incl. fp8 aliases (optimus_dl/core/dtype.py:10-132)."""

from __future__ import annotations

import torch

_ALIASES = {
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32, "f32": torch.float32,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16, "f16": torch.float16,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float64": torch.float64, "fp64": torch.float64, "double": torch.float64,
    "int8": torch.int8, "int16": torch.int16, "int32": torch.int32, "int64": torch.int64, "long": torch.int64,
    "uint8": torch.uint8, "bool": torch.bool,
    "float8_e4m3fn": torch.float8_e4m3fn, "fp8_e4m3": torch.float8_e4m3fn, "e4m3": torch.float8_e4m3fn,
    "float8_e4m3": torch.float8_e4m3fn, "fp8": torch.float8_e4m3fn, "fp8_e4m3fn": torch.float8_e4m3fn,
    "e4m3fn": torch.float8_e4m3fn,
    "float8_e5m2": torch.float8_e5m2, "fp8_e5m2": torch.float8_e5m2, "e5m2": torch.float8_e5m2,
    "e5m2fn": torch.float8_e5m2, "fp8_e5m2fn": torch.float8_e5m2, "float8_e5m2fn": torch.float8_e5m2,
}
_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def str_to_dtype(name: str | torch.dtype) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    key = str(name).strip().lower()
    if key.startswith("torch."):
        key = key[6:]
    if key not in _ALIASES:
        raise ValueError(f"Unsupported dtype string {name!r}; known: {sorted(_ALIASES)}")
    return _ALIASES[key]


def is_fp8_dtype(dtype: str | torch.dtype) -> bool:
    try:
        return str_to_dtype(dtype) in _FP8
    except ValueError:
        return False


def get_fp8_format_from_dtype(dtype: str | torch.dtype) -> str | None:
    """``"e4m3fn"`` / ``"e5m2"`` for the two fp8 types, ``None`` for every other dtype
    (optimus_dl/core/dtype.py:104-132)."""
    d = str_to_dtype(dtype)
    if d == torch.float8_e4m3fn:
        return "e4m3fn"
    if d == torch.float8_e5m2:
        return "e5m2"
    return None
