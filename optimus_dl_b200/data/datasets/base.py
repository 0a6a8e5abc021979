"""Dataset base node (optimus_dl/modules/data/datasets/base.py:12-68): a ``torchdata`` node with
``next`` / ``reset(state)`` / ``get_state``; ``load_state_dict`` is an alias of ``reset``."""

from __future__ import annotations

from typing import Any

from torchdata.nodes import BaseNode


class BaseDataset(BaseNode):
    def __init__(self, cfg: Any = None, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        super().__init__()
        self.cfg = cfg
        self.rank, self.world_size, self.seed = rank, world_size, seed

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)

    def get_state(self) -> dict[str, Any]:
        return {}

    def next(self) -> Any:
        raise NotImplementedError

    def load_state_dict(self, state: dict) -> None:
        self.reset(state)
