"""Transform base (optimus_dl/modules/data/transforms/base.py:13-147).

``transform.build(source) -> node``. Sub-classes' ``build`` is wrapped automatically so that, while a
pipeline profiler is active, the node they return is proxied for timing. ``MapperConfig`` holds
the knobs of ``torchdata.nodes.ParallelMapper`` based transforms.
"""

from __future__ import annotations

import functools
from dataclasses import dataclass
from typing import Any

from torchdata.nodes import BaseNode

from ..profiling import maybe_profile


class BaseTransform:
    def __init__(self, cfg: Any = None, **kwargs: Any):
        self.cfg = cfg

    def __init_subclass__(cls, **kwargs: Any) -> None:
        super().__init_subclass__(**kwargs)
        if "build" in cls.__dict__:
            orig = cls.__dict__["build"]

            @functools.wraps(orig)
            def wrapped(self, source: BaseNode, _orig=orig) -> BaseNode:
                node = _orig(self, source)
                return maybe_profile(node, type(self).__name__)

            cls.build = wrapped

    def build(self, source: BaseNode) -> BaseNode:
        raise NotImplementedError


@dataclass
class MapperConfig:
    num_workers: int = 4
    in_order: bool = True
    method: str = "thread"          # "thread" or "process"
    snapshot_frequency: int = 128
    prebatch: int | None = 32
    max_concurrent: int | None = None


@dataclass
class ProcessMapperConfig(MapperConfig):
    method: str = "process"


ThreadedMapperConfig = MapperConfig   # the reference's name for the thread-pool mapper settings
