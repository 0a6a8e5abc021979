"""Stand-in for `hydra`: only `hydra.utils.instantiate` / `get_class`, as the reference's lazy-instantiate helpers
import them. The reference arm of bench.py builds components from dataclass configs and does not use Hydra's CLI."""

from . import utils  # noqa: F401


def main(*_a, **_k):
    raise RuntimeError("hydra.main is not available in the bench.py reference arm")
