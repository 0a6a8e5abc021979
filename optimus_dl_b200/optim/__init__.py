"""Optimizers and the ``optimizer`` registry (``_name``: adamw, muon, soap, composite)."""

from ..core.bootstrap import bootstrap_module
from ..core.registry import make_registry

_OPTIMIZERS_REGISTRY, register_optimizer, build_optimizer = make_registry("optimizer")
bootstrap_module(__name__)
