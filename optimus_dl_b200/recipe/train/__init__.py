"""Train recipe and the ``train_recipe`` registry."""

from ...core.registry import make_registry
from .config import TrainConfig, TrainRecipeConfig

_TRAIN_RECIPE_REGISTRY, register_train_recipe, build_train_recipe = make_registry("train_recipe")

from .base import TrainRecipe  # noqa: E402

register_train_recipe("base", TrainConfig)(TrainRecipe)
