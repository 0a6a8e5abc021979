"""Typed readers for launcher environment variables (optimus_dl/core/env.py:15-138).

Every reader takes the reference's arguments -- ``(env, name)`` with an explicit mapping -- and also works without a
mapping, in which case ``os.environ`` is read and, for the rank / size helpers, the variables of the other common
launchers (Open MPI, Slurm) are tried after torchrun's.
"""

from __future__ import annotations

import os
from collections.abc import Mapping
from pathlib import Path
from typing import Any

import torch


class InvalidEnvironmentVariableError(ValueError):
    """``name`` holds the offending variable."""

    def __init__(self, name: str, message: str | None = None) -> None:
        super().__init__(message if message is not None else name)
        self.name = name


def _split(args: tuple, default_env: Mapping[str, str]) -> tuple[Mapping[str, str], tuple]:
    if args and isinstance(args[0], Mapping):
        return args[0], args[1:]
    return default_env, args


def get_int_from_env(*args: Any, allow_zero: bool | None = None, default: int | None = None) -> int | None:
    """``get_int_from_env(env, name, allow_zero=False)`` as in the reference (positive integers only unless
    ``allow_zero``), or ``get_int_from_env(names, default)`` over ``os.environ`` where ``names`` may be a list tried in
    order (any integer accepted)."""
    env, rest = _split(args, os.environ)
    reference_style = bool(args) and isinstance(args[0], Mapping)
    names = rest[0]
    if len(rest) > 1:
        if reference_style:
            allow_zero = bool(rest[1])
        else:
            default = rest[1]
    for n in [names] if isinstance(names, str) else list(names):
        v = env.get(n)
        if v is None or v == "":
            continue
        try:
            value = int(v)
        except ValueError:
            raise InvalidEnvironmentVariableError(
                n, f"The value of the `{n}` environment variable is expected to be an integer, but is '{v}' instead.") from None
        if reference_style or allow_zero is not None:
            low = 0 if allow_zero else 1
            if value < low:
                raise InvalidEnvironmentVariableError(
                    n, f"The value of the `{n}` environment variable is expected to be at least {low}, but is {value} instead.")
        return value
    return default


def get_path_from_env(*args: Any) -> Path | None:
    """``(env, name)`` or ``(name)``: the variable as a ``Path``; ``None`` when unset or empty."""
    env, rest = _split(args, os.environ)
    v = env.get(rest[0])
    if not v:
        return None
    try:
        return Path(v)
    except (ValueError, TypeError):
        raise InvalidEnvironmentVariableError(
            rest[0], f"The value of the `{rest[0]}` environment variable is expected to be a pathname, but is '{v}' instead.") from None


def get_device_from_env(*args: Any) -> torch.device | None:
    """``(env, name)`` or ``(name)``: the variable as a ``torch.device``; ``None`` when unset."""
    env, rest = _split(args, os.environ)
    v = env.get(rest[0])
    if v is None:
        return None
    try:
        return torch.device(v)
    except (RuntimeError, ValueError):
        raise InvalidEnvironmentVariableError(
            rest[0], f"The value of the `{rest[0]}` environment variable is expected to specify a PyTorch device, but is '{v}' "
                     "instead.") from None


def _first(env: Mapping[str, str] | None, names: list[str], allow_zero: bool, fallback: int) -> int:
    if env is not None:                       # reference call: torchrun's variable only, range-checked
        value = get_int_from_env(env, names[0], allow_zero)
        return fallback if value is None else value
    value = get_int_from_env(names, None)
    return fallback if value is None else value


def get_world_size(env: Mapping[str, str] | None = None) -> int:
    return _first(env, ["WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "SLURM_NTASKS"], False, 1)


def get_rank(env: Mapping[str, str] | None = None) -> int:
    return _first(env, ["RANK", "OMPI_COMM_WORLD_RANK", "SLURM_PROCID"], True, 0)


def get_local_rank(env: Mapping[str, str] | None = None) -> int:
    return _first(env, ["LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID"], True, 0)


def get_local_world_size(env: Mapping[str, str] | None = None) -> int:
    if env is not None:
        return _first(env, ["LOCAL_WORLD_SIZE"], False, 1)
    value = get_int_from_env(["LOCAL_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_SIZE"], None)
    return value if value else get_world_size()
