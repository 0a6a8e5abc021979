"""Data builder (optimus_dl/recipe/train/builders/data_builder.py:51-165).

Data is sharded by *data-parallel* rank (tensor-parallel peers read identical batches) and each
rank derives its own seed from ``data_seed``. Evaluation loaders are resettable: iterating them
again restarts the underlying pipeline."""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

import torch
import torchdata.nodes as tn

from ....core.registry import RegistryConfig, make_registry
from ....data import build_data_pipeline, build_data_pipeline_dict

logger = logging.getLogger(__name__)


@dataclass
class DataBuilderConfig(RegistryConfig):
    pass


def per_rank_seed(seed: int, rank: int, world_size: int) -> int:
    g = torch.Generator()
    g.manual_seed(int(seed) + world_size * 10000 + rank)
    # the same draw as optimus_dl/recipe/train/builders/data_builder.py:51-57, so that one ``data_seed`` gives one
    # data order in both code bases
    return int(torch.randint(0, 2**32, (1,), generator=g).item())


class LoaderIterResettable:
    """``iter(x)`` restarts the pipeline; the current iterator's state is reachable for checkpoints."""

    def __init__(self, node: Any):
        self.node = node
        self.loader = tn.Loader(node, restart_on_stop_iteration=True)
        self._it = None

    def __iter__(self):
        self._it = iter(self.loader)
        return self._it

    def state_dict(self) -> dict:
        return self.loader.state_dict()

    def load_state_dict(self, state: dict) -> None:
        self.loader.load_state_dict(state)


class DataBuilder:
    def __init__(self, cfg: Any = None, data_config: Any = None, data_seed: int = 42, **kwargs: Any):
        self.cfg, self.data_config, self.data_seed = cfg, data_config, data_seed

    def _kwargs(self, collective: Any, device: Any) -> dict[str, Any]:
        rank = collective.dp_rank if collective is not None else 0
        world = collective.dp_world_size if collective is not None else 1
        # ``seed`` differs per rank (shuffle buffers, sampling); ``global_seed`` is the same everywhere, for what the
        # ranks must agree on (a sharded dataset's permutation and offset: with per-rank seeds the ranks' shares of a
        # shuffled corpus would overlap)
        return dict(rank=rank, world_size=world, seed=per_rank_seed(self.data_seed, rank, world), device=device,
                    global_seed=int(self.data_seed))

    def build_train_data(self, collective: Any = None, device: Any = None, **kwargs: Any):
        cfg = self.data_config.get("train_datasets") if self.data_config is not None else None
        if cfg is None:
            return None
        pipe = build_data_pipeline(cfg, profile_name="train", eval_pipeline=False, **self._kwargs(collective, device), **kwargs)
        return pipe._replace(dataloader=tn.Loader(pipe.dataloader, restart_on_stop_iteration=False))

    def build_eval_data(self, collective: Any = None, device: Any = None, **kwargs: Any) -> dict[str, Any]:
        cfg = self.data_config.get("eval_datasets") if self.data_config is not None else None
        if not cfg:
            return {}
        pipes = {k: build_data_pipeline(v, profile_name=f"eval-{k}", eval_pipeline=True, **self._kwargs(collective, device),
                                        **kwargs) for k, v in cfg.items()}
        return {k: p._replace(dataloader=LoaderIterResettable(p.dataloader)) for k, p in pipes.items() if p is not None}


_R, register_data_builder, build_data_builder = make_registry("data_builder")
register_data_builder("base", DataBuilderConfig)(DataBuilder)
