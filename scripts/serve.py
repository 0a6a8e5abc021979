"""Serve a model over HTTP (OpenAI-style completions and chat completions).

    python scripts/serve.py --config-name=char_shakespeare common.checkpoint_path=outputs/run/metadata_latest.pt
    curl -s http://127.0.0.1:8000/v1/completions -d '{"prompt": "ROMEO:", "max_tokens": 64, "temperature": 0.8}'
"""

import logging
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.core import compose, conf  # noqa: E402
from optimus_dl_b200.core.config_utils import non_resolving_instantiate  # noqa: E402
from optimus_dl_b200.core.log import setup_logging  # noqa: E402
from optimus_dl_b200.core.multiprocess import finalize_process  # noqa: E402
from optimus_dl_b200.recipe.serve import ServeConfig, ServeRecipe  # noqa: E402

logger = logging.getLogger(__name__)


@compose.main(config_path="../configs/serve", config_name="tinyllama")
def serve(cfg_raw):
    setup_logging()
    cfg = conf.merge(conf.create(ServeConfig()), non_resolving_instantiate(cfg_raw))
    recipe = ServeRecipe(cfg)
    try:
        recipe.run()
    finally:
        finalize_process()


if __name__ == "__main__":
    serve()
