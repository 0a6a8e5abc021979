"""Per-rank mid-evaluation state so an interrupted evaluation resumes where it stopped
(optimus_dl/modules/checkpoint/eval_checkpoint_manager.py:17-198).

Files: ``{output}/eval_checkpoints_iter_{N}/{eval_name}_rank_{r}.pt`` holding the meter group of that
evaluation, the dataloader state and the number of batches already processed. Writes are atomic
(tmp + rename); directories of other iterations are removed on cleanup."""

from __future__ import annotations

import os
import shutil
from pathlib import Path
from typing import Any

import torch

from ..metrics import base as meters


class EvaluationCheckpointManager:
    def __init__(self, output_path: str, rank: int = 0):
        self.root = Path(output_path)
        self.rank = rank

    def _dir(self, iteration: int) -> Path:
        return self.root / f"eval_checkpoints_iter_{iteration}"

    def get_eval_checkpoints_dir(self, iteration: int) -> Path:
        """Directory that holds the mid-evaluation states of ``iteration``."""
        return self._dir(iteration)

    def _file(self, iteration: int, eval_name: str) -> Path:
        safe = eval_name.replace("/", "_")
        return self._dir(iteration) / f"{safe}_rank_{self.rank}.pt"

    def save_iteration_state(self, iteration: int, eval_name: str, group_name: str, dataloader_state: Any,
                             processed: int) -> None:
        d = self._dir(iteration)
        d.mkdir(parents=True, exist_ok=True)
        g = meters.get_group(group_name)
        state = {"meters": g.state_dict() if g is not None else None, "dataloader": dataloader_state,
                 "eval_iterations_processed": processed, "iteration": iteration}
        path = self._file(iteration, eval_name)
        tmp = path.with_suffix(".pt.tmp")
        torch.save(state, tmp)
        os.replace(tmp, path)

    def load_iteration_state(self, iteration: int, eval_name: str, group_name: str) -> dict[str, Any] | None:
        path = self._file(iteration, eval_name)
        if not path.exists():
            return None
        state = torch.load(path, map_location="cpu", weights_only=False)
        if state.get("meters") is not None:
            meters.load_state_dict({group_name: state["meters"]})
        return state

    def cleanup(self, iteration: int | None = None, exclude_iteration: int | None = None) -> None:
        """Remove the states of ``iteration``, or of every iteration except ``exclude_iteration``."""
        if not self.root.exists():
            return
        if iteration is not None:
            shutil.rmtree(self._dir(iteration), ignore_errors=True)
            return
        for d in self.root.glob("eval_checkpoints_iter_*"):
            if exclude_iteration is not None and d.name == f"eval_checkpoints_iter_{exclude_iteration}":
                continue
            shutil.rmtree(d, ignore_errors=True)
