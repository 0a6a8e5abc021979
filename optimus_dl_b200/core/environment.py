"""Named environment knobs (optimus_dl/core/environment.py:6-33)."""

from __future__ import annotations

import os
from typing import Any, Callable


class EnvironmentVariable:
    def __init__(self, name: str, default: Any = None, cast: Callable[[str], Any] = str):
        self.name, self.default, self.cast = name, default, cast

    def get(self) -> Any:
        v = os.environ.get(self.name)
        if v is None:
            return self.default
        if self.cast is bool:
            return v.strip().lower() in ("1", "true", "yes", "on")
        return self.cast(v)

    def is_set(self) -> bool:
        return self.name in os.environ

    def __bool__(self) -> bool:
        return bool(self.get())


OPTIMUS_DEBUG = EnvironmentVariable("OPTIMUS_DEBUG", False, bool)
OPTIMUS_EXIT_TIMEOUT = EnvironmentVariable("OPTIMUS_EXIT_TIMEOUT", 30.0, float)
