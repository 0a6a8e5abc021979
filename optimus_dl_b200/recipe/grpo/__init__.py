"""GRPO reinforcement-learning recipe; registered as ``grpo_recipe`` / ``base``."""

from ...core.registry import make_registry
from .base import GRPORecipe
from .config import GRPOConfig
from .rewards import build_reward, register_reward

_R, register_grpo_recipe, build_grpo_recipe = make_registry("grpo_recipe")
register_grpo_recipe("base", GRPOConfig)(GRPORecipe)

__all__ = ["GRPORecipe", "GRPOConfig", "build_grpo_recipe", "build_reward", "register_reward"]
