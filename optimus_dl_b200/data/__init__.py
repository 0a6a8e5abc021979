"""Source -> transform data pipelines on ``torchdata.nodes`` (optimus_dl/modules/data/__init__.py:36-131).

``build_data_pipeline(cfg, profile_name, **kw)`` builds the source from the ``dataset`` registry,
wraps it in a ``LoggingDataNode``, optionally attaches the pipeline profiler and applies
``transform.build(node)``. ``kw`` (``rank``, ``world_size``, ``seed``, ``device``) reach every dataset and
transform constructor.
"""

from __future__ import annotations

import logging
from typing import Any, NamedTuple

from torchdata.nodes import BaseNode

from .datasets import build_dataset
from .datasets.base import BaseDataset
from .profiling import PipelineProfiler, ProfilingProxyNode, scope_profiler
from .transforms import build_transform

logger = logging.getLogger(__name__)


class DataPipeline(NamedTuple):
    datasets: Any
    dataloader: Any


class EvalDataPipeline(NamedTuple):
    datasets: Any
    dataloader: Any
    eval_freq: int | None
    eval_iterations: int | None
    eval_guaranteed_same_batches: bool | None
    eval_checkpointing: int | None


class LoggingDataNode(BaseDataset):
    """Logs resets and delegates everything else to the wrapped source."""

    def __init__(self, name: str, source: BaseNode):
        super().__init__(None)
        self.name = name
        self.source = source

    def reset(self, initial_state: dict | None = None):
        logger.info("Resetting data node %s (resume=%s)", self.name, initial_state is not None)
        super().reset(initial_state)
        self.source.reset(initial_state)

    def get_state(self) -> dict[str, Any]:
        return self.source.state_dict()

    def next(self):
        return next(self.source)

    def __repr__(self) -> str:
        return f"LoggingDataNode(name={self.name}, source={self.source!r})"


_EVAL_KEYS = ("eval_freq", "eval_iterations", "eval_guaranteed_same_batches", "eval_checkpointing")


def _get(cfg: Any, key: str, default: Any = None) -> Any:
    if cfg is None:
        return default
    if isinstance(cfg, dict) or hasattr(cfg, "get"):
        try:
            return cfg.get(key, default)
        except Exception:
            pass
    return getattr(cfg, key, default)


def _has(cfg: Any, key: str) -> bool:
    try:
        return key in cfg
    except TypeError:
        return hasattr(cfg, key)


def build_data_pipeline(cfg: Any, profile_name: str | None = None, eval_pipeline: bool | None = None, **kwargs: Any):
    if cfg is None:
        return None
    dataset = build_dataset(_get(cfg, "source"), **kwargs)
    dataset_class = type(dataset).__name__
    dataset = LoggingDataNode(name=profile_name or repr(dataset), source=dataset)
    pipeline: Any = dataset
    profiler = None
    if _get(cfg, "profile", False):
        profiler = PipelineProfiler(name=profile_name or repr(dataset), report_freq=_get(cfg, "report_freq", 100))
        pipeline = ProfilingProxyNode(pipeline, name=dataset_class, profiler=profiler)
    with scope_profiler(profiler):
        tcfg = _get(cfg, "transform")
        if tcfg is not None:
            pipeline = build_transform(tcfg, **kwargs).build(pipeline)
        if isinstance(pipeline, ProfilingProxyNode):
            pipeline._is_root = True
    assert isinstance(pipeline, BaseNode), f"transform produced {type(pipeline).__name__}, not a data node"
    is_eval = eval_pipeline if eval_pipeline is not None else any(_has(cfg, k) for k in _EVAL_KEYS)
    if is_eval:
        return EvalDataPipeline(dataset, pipeline, *[_get(cfg, k) for k in _EVAL_KEYS])
    return DataPipeline(dataset, pipeline)


def build_data_pipeline_dict(cfg: Any, profile_name: str, **kwargs: Any) -> dict[str, Any]:
    return {k: build_data_pipeline(v, profile_name=f"{profile_name}-{k}", **kwargs) for k, v in (cfg or {}).items()}
