"""GRPO reinforcement-learning entry point.

    torchrun --nproc_per_node=gpu scripts/grpo.py
    python scripts/grpo.py model=llama2-lite grpo.num_prompts=8 grpo.max_new_tokens=32 common.use_gpu=false
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.core import compose  # noqa: E402
from optimus_dl_b200.core.config_utils import non_resolving_instantiate  # noqa: E402
from optimus_dl_b200.core.log import setup_logging  # noqa: E402
from optimus_dl_b200.core.multiprocess import finalize_process  # noqa: E402
from optimus_dl_b200.core.registry import build  # noqa: E402


@compose.main(config_path="../configs/grpo", config_name="default")
def main(cfg_raw):
    setup_logging()
    recipe = build("grpo_recipe", non_resolving_instantiate(cfg_raw))
    try:
        recipe.run()
    finally:
        finalize_process()
    return recipe


if __name__ == "__main__":
    main()
