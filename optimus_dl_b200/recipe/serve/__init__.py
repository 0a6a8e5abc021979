from .base import ServeRecipe
from .config import ServeConfig

__all__ = ["ServeRecipe", "ServeConfig"]
