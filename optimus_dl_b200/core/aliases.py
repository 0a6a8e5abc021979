"""Second names for modules whose path differs from the reference's tree.

Code written against the reference imports ``optimus_dl.modules.<x>`` and ``optimus_dl.core.<y>``; here the same
components live under ``optimus_dl_b200.<x>`` and ``optimus_dl_b200.core.<y>``, so a port is one prefix substitution
(``optimus_dl.modules.`` -> ``optimus_dl_b200.``, then ``optimus_dl.`` -> ``optimus_dl_b200.``) -- except for three
places where this package chose another layout:

=================================================  ==========================================
reference path (after the substitution)            module here
=================================================  ==========================================
``optimus_dl_b200.model[.<sub>]``                  ``optimus_dl_b200.models[.<sub>]``
``optimus_dl_b200.distributed[.base|config|..]``   ``optimus_dl_b200.parallel.collective``
``optimus_dl_b200.core.omegaconf_utils``           ``optimus_dl_b200.core.config_utils``
=================================================  ==========================================

``install()`` puts a finder in front of ``sys.meta_path`` that answers imports of the left-hand names with the very
module objects of the right-hand ones (no second execution, so registries and classes stay unique). Reference
layout: optimus_dl/modules/model/, optimus_dl/modules/distributed/{__init__,base,config,fake,mesh}.py,
optimus_dl/core/omegaconf_utils.py.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import sys
import types

_ROOT = __name__.split(".")[0]

# alias prefix -> (real module, whether sub-names map onto sub-modules of the real package)
_PREFIXES = {
    f"{_ROOT}.model": (f"{_ROOT}.models", True),
    f"{_ROOT}.distributed": (f"{_ROOT}.parallel.collective", False),
    f"{_ROOT}.core.omegaconf_utils": (f"{_ROOT}.core.config_utils", False),
}


def _resolve(fullname: str) -> tuple[str, bool] | None:
    """``(real module name, synthesise_package)`` for an aliased name, else None."""
    for alias, (real, mirrors_tree) in _PREFIXES.items():
        if fullname == alias:
            return real, not mirrors_tree and alias.endswith(".distributed")
        if fullname.startswith(alias + "."):
            rest = fullname[len(alias) + 1:]
            return (f"{real}.{rest}", False) if mirrors_tree else (real, False)
    return None


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        hit = _resolve(fullname)
        if hit is None:
            return None
        real_name, as_package = hit
        try:
            real = importlib.import_module(real_name)
        except ModuleNotFoundError:
            return None
        spec = importlib.machinery.ModuleSpec(fullname, self, is_package=as_package or hasattr(real, "__path__"))
        spec._alias_target = (real, as_package)  # noqa: SLF001 - carried to create_module
        return spec

    def create_module(self, spec):
        real, as_package = spec._alias_target  # noqa: SLF001
        if not as_package:
            return real
        # a single module standing in for a package with sub-modules: same names, plus an (empty) search path so
        # that ``import <alias>.<sub>`` reaches this finder again
        pkg = types.ModuleType(spec.name, real.__doc__)
        pkg.__dict__.update({k: v for k, v in vars(real).items() if not (k.startswith("__") and k.endswith("__"))})
        pkg.__path__ = []
        return pkg

    def exec_module(self, module):
        return None


_finder: _AliasFinder | None = None


def install() -> None:
    """Idempotent; called by the package on import."""
    global _finder
    if _finder is None:
        _finder = _AliasFinder()
        sys.meta_path.insert(0, _finder)
