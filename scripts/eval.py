"""Evaluate a checkpoint with the lm_eval harness.

    python scripts/eval.py common.checkpoint_path=outputs/run common.tokenizer._name=char_tokenize
    python scripts/eval.py --config-name=quick common.checkpoint_path=outputs/run lm_eval.tasks=[arc_easy]
"""

import logging
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.core import compose, conf  # noqa: E402
from optimus_dl_b200.core.config_utils import non_resolving_instantiate  # noqa: E402
from optimus_dl_b200.core.log import setup_logging  # noqa: E402
from optimus_dl_b200.core.multiprocess import finalize_process  # noqa: E402
from optimus_dl_b200.recipe.eval import EvalConfig, EvalRecipe  # noqa: E402

logger = logging.getLogger(__name__)


@compose.main(config_path="../configs/eval", config_name="default")
def evaluate(cfg_raw):
    setup_logging()
    cfg = conf.merge(conf.create(EvalConfig()), non_resolving_instantiate(cfg_raw))
    recipe = EvalRecipe(cfg)
    try:
        results = recipe.run()
        for task, metrics in (results.get("results") or {}).items():
            print(task, {k: round(v, 4) for k, v in metrics.items() if isinstance(v, float)})
        return results
    finally:
        finalize_process()


if __name__ == "__main__":
    evaluate()
