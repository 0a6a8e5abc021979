"""Offline metric evaluation recipe; registered as ``metrics_recipe`` / ``base``."""

from ...core.registry import make_registry
from .base import MetricsRecipe
from .config import MetricsConfig

_R, register_metrics_recipe, build_metrics_recipe = make_registry("metrics_recipe")
register_metrics_recipe("base", MetricsConfig)(MetricsRecipe)

__all__ = ["MetricsRecipe", "MetricsConfig", "build_metrics_recipe"]
