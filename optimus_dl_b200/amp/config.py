"""Re-export of the AMP configs (optimus_dl/modules/amp/config.py)."""

from ..optim.config import AmpConfig, Fp8Config, OptimizationConfig  # noqa: F401
