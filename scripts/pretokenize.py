"""Tokenise a dataset into sharded ``.npy`` files.

    python scripts/pretokenize.py dataset.repo_id=roneneldan/TinyStories output.dir=data/tinystories
    python scripts/pretokenize.py dataset.repo_id=/data/my_corpus dataset.file_pattern='*.jsonl' tokenizer=llama3
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.core import compose, conf  # noqa: E402
from optimus_dl_b200.core.config_utils import non_resolving_instantiate  # noqa: E402
from optimus_dl_b200.core.log import setup_logging  # noqa: E402
from optimus_dl_b200.recipe.pretokenize import DataPrepConfig, DataPrepRecipe  # noqa: E402


@compose.main(config_path="../configs/prepare_data", config_name="default")
def main(cfg_raw):
    setup_logging()
    cfg = conf.merge(conf.create(DataPrepConfig()), non_resolving_instantiate(cfg_raw))
    DataPrepRecipe(cfg).run()


if __name__ == "__main__":
    main()
