"""Evaluate a model with the internal metric engine (no training).

    python scripts/metrics.py --config-name=tinystories_test common.checkpoint_path=outputs/run
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.core import compose  # noqa: E402
from optimus_dl_b200.core.config_utils import non_resolving_instantiate  # noqa: E402
from optimus_dl_b200.core.log import setup_logging  # noqa: E402
from optimus_dl_b200.core.multiprocess import finalize_process  # noqa: E402
from optimus_dl_b200.core.registry import build  # noqa: E402


@compose.main(config_path="../configs/metrics", config_name="default")
def metrics(cfg_raw):
    setup_logging()
    cfg = non_resolving_instantiate(cfg_raw)
    recipe = build("metrics_recipe", cfg)
    try:
        results = recipe.run()
        for name, vals in results.items():
            print(name, {k: v for k, v in vals.items() if isinstance(v, (int, float))})
        return results
    finally:
        finalize_process()


if __name__ == "__main__":
    metrics()
