"""Mixed precision: autocast contexts and the FP8 recipe objects.

Exports what the reference's package exports (optimus_dl/modules/amp/__init__.py): the config dataclasses eagerly,
the FP8 helpers on first access (``amp.fp8`` imports kernels and configs that import this package).
"""

from .config import AmpConfig, Fp8Config, OptimizationConfig  # noqa: F401

_FP8_EXPORTS = ("Fp8Format", "Fp8RecipeType", "FP8Recipe", "Fp8RecipeConfig", "create_fp8_recipe", "fp8_autocast",
                "fp8_backward", "get_fp8_format_from_string", "get_fp8_recipe_type_from_string",
                "get_transformer_engine_version", "is_transformer_engine_available")


def __getattr__(name: str):
    if name in _FP8_EXPORTS:
        from . import fp8

        return getattr(fp8, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
