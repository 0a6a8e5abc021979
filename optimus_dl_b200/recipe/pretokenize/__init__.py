from .config import DataPrepConfig
from .recipe import DataPrepRecipe

__all__ = ["DataPrepRecipe", "DataPrepConfig"]
