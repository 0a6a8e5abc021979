"""Data preparation recipe: dataset files -> tokenised, sharded ``.npy`` dataset with ``index.json``
(optimus_dl/recipe/pretokenize/recipe.py:28-160). A progress checkpoint is written whenever a shard
is closed and on Ctrl-C; running the same command again resumes from it."""

from __future__ import annotations

import logging
from pathlib import Path
from typing import Any

import numpy as np

from ...core import conf
from ...core.log import tqdm
from ...tokenizer import build_tokenizer
from .checkpoint import CheckpointManager, CheckpointState
from .processor import TokenProcessor
from .sharder import Sharder
from .source import FileFinder

logger = logging.getLogger(__name__)


class DataPrepRecipe:
    def __init__(self, config: Any):
        self.config = config
        self.output_dir = Path(str(config.output.dir))
        self.output_dir.mkdir(parents=True, exist_ok=True)
        self.sharder = Sharder(config.output, config.processing)
        self.checkpointer = CheckpointManager(self.output_dir)
        self._check_tokenizer()

    def _check_tokenizer(self) -> None:
        tokenizer = build_tokenizer(self.config.tokenizer)
        limit = np.iinfo(self.sharder.dtype).max
        if tokenizer.vocab_size > limit:
            raise ValueError(f"Tokenizer vocab size ({tokenizer.vocab_size}) exceeds the maximum value for the chosen "
                             f"dtype '{np.dtype(self.sharder.dtype).name}' ({limit}). Please use a larger dtype (e.g., uint32).")

    def _state(self, processor: TokenProcessor) -> CheckpointState:
        return CheckpointState(processor_state=processor.get_state(), sharder_state=self.sharder.get_state())

    def run(self) -> None:
        files = FileFinder(self.config.dataset, int(self.config.processing.seed)).get_files()
        if not files:
            logger.error("No files found to process. Aborting.")
            return
        processor = TokenProcessor(files, self.config)
        checkpoint = self.checkpointer.load()
        if checkpoint is not None:
            logger.info("resuming from a checkpoint (file %d)", checkpoint.processor_state.get("file_idx", 0))
            processor.load_state(checkpoint.processor_state)
            self.sharder.load_state(checkpoint.sharder_state)
        bar = tqdm(total=len(files), desc="Files", unit="file", initial=processor.progress)
        seen = processor.progress
        try:
            for doc in processor:
                if processor.progress > seen:
                    bar.update(processor.progress - seen)
                    seen = processor.progress
                if self.sharder.add(doc):
                    self.checkpointer.save(self._state(processor))
            self.sharder.finalize(self._final_config())
            self.checkpointer.clean()
        except KeyboardInterrupt:
            logger.info("interrupted: saving a checkpoint; run the same command again to resume")
            self.checkpointer.save(self._state(processor))
        finally:
            processor.close()
            bar.close()

    def _final_config(self) -> dict[str, Any]:
        t = self.config.tokenizer
        return {"dataset": str(self.config.dataset.repo_id), "split": str(self.config.dataset.split),
                "dtype": str(self.config.processing.dtype),
                "tokenizer": conf.to_container(t, resolve=True) if conf.is_config(t) else dict(t)}
