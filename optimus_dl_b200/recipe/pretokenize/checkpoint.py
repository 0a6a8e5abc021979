"""Atomic progress checkpoints of the data preparation recipe
(optimus_dl/recipe/pretokenize/checkpoint.py:14-73): ``checkpoint.pkl`` written via a temporary file."""

from __future__ import annotations

import logging
import os
import pickle
from dataclasses import dataclass
from pathlib import Path
from typing import Any

logger = logging.getLogger(__name__)


@dataclass
class CheckpointState:
    processor_state: dict[str, Any]
    sharder_state: dict[str, Any]


class CheckpointManager:
    def __init__(self, output_dir: Path):
        self.checkpoint_path = Path(output_dir) / "checkpoint.pkl"
        self.tmp_path = Path(output_dir) / "checkpoint.tmp"

    def save(self, state: CheckpointState) -> None:
        with open(self.tmp_path, "wb") as f:
            pickle.dump(state, f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(self.tmp_path, self.checkpoint_path)

    def load(self) -> CheckpointState | None:
        if not self.checkpoint_path.exists():
            return None
        try:
            with open(self.checkpoint_path, "rb") as f:
                state = pickle.load(f)
        except Exception as err:  # noqa: BLE001
            logger.warning("failed to load checkpoint (%s); starting from scratch", err)
            return None
        if not isinstance(state, CheckpointState):
            logger.warning("checkpoint file is invalid or outdated, ignoring")
            return None
        return state

    def clean(self) -> None:
        if self.checkpoint_path.exists():
            self.checkpoint_path.unlink()
