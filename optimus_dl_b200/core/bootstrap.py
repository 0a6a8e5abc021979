"""Import every module of a package so that ``@register_*`` decorators run.

Mirrors optimus_dl/core/bootstrap.py:6-69: non-underscore modules and sub-packages are
imported; names containing ``test_``, ``tests``, ``__pycache__`` or ``.pyc`` are skipped.
"""

from __future__ import annotations

import importlib
import logging
import os

logger = logging.getLogger(__name__)
_SKIP = ("test_", "tests", "__pycache__", ".pyc")


def bootstrap_module(module_name: str, path: str | None = None) -> list[str]:
    """Import all public modules under ``module_name``; returns the imported names."""
    mod = importlib.import_module(module_name)
    base = path or os.path.dirname(mod.__file__ or "")
    imported: list[str] = []
    for entry in sorted(os.listdir(base)):
        if entry.startswith("_") or entry.startswith(".") or any(s in entry for s in _SKIP):
            continue
        full = os.path.join(base, entry)
        if os.path.isdir(full):
            if os.path.exists(os.path.join(full, "__init__.py")):
                name = f"{module_name}.{entry}"
            else:
                continue
        elif entry.endswith(".py"):
            name = f"{module_name}.{entry[:-3]}"
        else:
            continue
        importlib.import_module(name)
        imported.append(name)
        if os.path.isdir(full):
            # sub-packages are walked too, so nested implementation folders register themselves
            imported.extend(bootstrap_module(name, full))
    return imported
