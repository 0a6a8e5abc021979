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
    """``rank`` is the default rank of the file name; a ``collective`` given to a call overrides it, so one
    manager object serves every rank of a spawned group."""

    def __init__(self, output_path: str | Path, rank: int = 0):
        self.output_path = Path(output_path)
        self.rank = rank

    @property
    def root(self) -> Path:
        return self.output_path

    def get_eval_checkpoints_dir(self, iteration: int) -> Path:
        """Directory that holds the mid-evaluation states of ``iteration``."""
        return self.output_path / f"eval_checkpoints_iter_{iteration}"

    def _file(self, iteration: int, eval_name: str, collective: Any = None) -> tuple[Path, int]:
        rank = collective.rank if collective is not None else self.rank
        return self.get_eval_checkpoints_dir(iteration) / f"{eval_name.replace('/', '_')}_rank_{rank}.pt", rank

    def save_iteration_state(self, iteration: int, eval_name: str, dataloader_state: Any, group_name: str,
                             collective: Any = None, eval_iterations_processed: int = 0) -> None:
        """Write this rank's state: the meters of ``group_name``, the dataloader state and the batch count."""
        path, rank = self._file(iteration, eval_name, collective)
        path.parent.mkdir(parents=True, exist_ok=True)
        g = meters.get_group(group_name)
        if g is None:
            raise AssertionError(f"Group {group_name} not found in meters state")
        state = {"iteration": iteration, "eval_name": eval_name, "group_name": group_name, "rank": rank,
                 "meters_state": g.state_dict(), "dataloader_state": dataloader_state,
                 "eval_iterations_processed": eval_iterations_processed}
        tmp = path.with_suffix(f".tmp{os.getpid()}")
        torch.save(state, tmp)
        os.replace(tmp, path)

    def read_iteration_state(self, iteration: int, eval_name: str, collective: Any = None) -> dict[str, Any] | None:
        """The saved dictionary of this rank, or ``None``; restores nothing."""
        path, _ = self._file(iteration, eval_name, collective)
        if not path.exists():
            return None
        return torch.load(path, map_location="cpu", weights_only=False)

    def load_iteration_state(self, iteration: int, eval_name: str, group_name: str, eval_iter: Any = None,
                             collective: Any = None) -> int:
        """Restore meters and, through ``eval_iter.reset(state)`` (``load_state_dict`` where there is no ``reset``),
        the dataloader; returns the number of batches already processed, 0 when nothing was saved."""
        assert iteration is not None, "Iteration must be provided to load evaluation checkpoint"
        state = self.read_iteration_state(iteration, eval_name, collective)
        if state is None:
            return 0
        _, rank = self._file(iteration, eval_name, collective)
        for key, want in (("iteration", iteration), ("eval_name", eval_name), ("rank", rank), ("group_name", group_name)):
            assert state[key] == want, f"Checkpoint {key} mismatch: expected {want}, got {state[key]}"
        meters.load_state_dict({group_name: state["meters_state"]})
        if eval_iter is not None and state.get("dataloader_state") is not None:
            if hasattr(eval_iter, "reset"):
                eval_iter.reset(state["dataloader_state"])
            else:
                assert hasattr(eval_iter, "load_state_dict"), "eval_iter needs reset(state) or load_state_dict(state)"
                eval_iter.load_state_dict(state["dataloader_state"])
        return int(state["eval_iterations_processed"])

    def cleanup(self, iteration: int | None = None, exclude_iteration: int | None = None) -> None:
        """Remove the states of ``iteration``, or of every iteration except ``exclude_iteration``."""
        assert not (iteration is not None and exclude_iteration is not None), \
            "Cannot specify both iteration and exclude_iteration"
        if not self.output_path.exists():
            return
        if iteration is not None:
            shutil.rmtree(self.get_eval_checkpoints_dir(iteration), ignore_errors=True)
            return
        for d in self.output_path.glob("eval_checkpoints_iter_*"):
            if exclude_iteration is not None and d.name == f"eval_checkpoints_iter_{exclude_iteration}":
                continue
            shutil.rmtree(d, ignore_errors=True)
