"""Loss functions and the ``criterion`` registry."""

from ..core.bootstrap import bootstrap_module
from ..core.registry import make_registry
from .base import BaseCriterion

_CRITERION_REGISTRY, register_criterion, build_criterion = make_registry("criterion", BaseCriterion)
bootstrap_module(__name__)
