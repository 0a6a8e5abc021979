"""Typed readers for the launcher's environment (optimus_dl/core/env.py:15-138)."""

from __future__ import annotations

import os


class InvalidEnvironmentVariableError(ValueError):
    pass


def get_int_from_env(names: str | list[str], default: int | None = None) -> int | None:
    for n in [names] if isinstance(names, str) else names:
        v = os.environ.get(n)
        if v is None or v == "":
            continue
        try:
            return int(v)
        except ValueError:
            raise InvalidEnvironmentVariableError(f"{n}={v!r} is not an integer") from None
    return default


def get_world_size() -> int:
    return get_int_from_env(["WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "SLURM_NTASKS"], 1) or 1


def get_rank() -> int:
    return get_int_from_env(["RANK", "OMPI_COMM_WORLD_RANK", "SLURM_PROCID"], 0) or 0


def get_local_rank() -> int:
    return get_int_from_env(["LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID"], 0) or 0


def get_local_world_size() -> int:
    return get_int_from_env(["LOCAL_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_SIZE"], None) or get_world_size()
