from .base import EvalRecipe
from .config import EvalConfig

__all__ = ["EvalRecipe", "EvalConfig"]
