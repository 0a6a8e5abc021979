"""Training entry point.

    python scripts/train.py                                   # configs/train/train_llama.yaml
    python scripts/train.py --config-name=train_llama_shakespeare common.use_gpu=false
    torchrun --nproc_per_node=gpu scripts/train.py model=llama2-1b optimization.acc_steps=4
    python scripts/train.py -m optimization.optimizer.lr=1e-3,1e-4    # sweep

Config composition, overrides and ``_target_`` instantiation follow Hydra's grammar
(``optimus_dl_b200/core/compose.py``)."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.core import compose  # noqa: E402
from optimus_dl_b200.core.config_utils import non_resolving_instantiate  # noqa: E402
from optimus_dl_b200.core.log import setup_logging  # noqa: E402
from optimus_dl_b200.core.multiprocess import finalize_process  # noqa: E402
from optimus_dl_b200.core.registry import build  # noqa: E402
from optimus_dl_b200.recipe.train import TrainRecipe  # noqa: E402


@compose.main(config_path="../configs/train", config_name="train_llama")
def train(cfg_raw):
    setup_logging()
    cfg = non_resolving_instantiate(cfg_raw)
    recipe = build("train_recipe", cfg)
    assert isinstance(recipe, TrainRecipe)
    try:
        recipe.run()
    finally:
        finalize_process()
    return recipe


if __name__ == "__main__":
    train()
