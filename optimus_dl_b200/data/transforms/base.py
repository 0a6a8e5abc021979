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


def adopt_saved_cfg(own: Any, saved: Any) -> Any:
    """Configuration of a node restored from a checkpoint: the saved values win (a run continues with the settings
    it was started with, as in the reference), for the fields this node knows; fields the saved object does not have
    (it may come from another version, or from the reference) keep their current value."""
    if saved is None or saved is own:
        return own
    import copy
    import dataclasses

    def has(obj: Any, k: str) -> bool:
        try:
            return k in obj
        except TypeError:
            return hasattr(obj, k)

    def get(obj: Any, k: str) -> Any:
        try:
            return obj[k]
        except (TypeError, KeyError, AttributeError):
            return getattr(obj, k)

    out = copy.copy(own)
    names = [f.name for f in dataclasses.fields(own)] if dataclasses.is_dataclass(own) else list(own.keys())
    for k in names:
        if k.startswith("_") or not has(saved, k):
            continue
        try:
            v = get(saved, k)
        except Exception:  # noqa: BLE001 - a missing mandatory value in the saved object
            continue
        if dataclasses.is_dataclass(own):
            setattr(out, k, v)
        else:
            out[k] = v
    return out


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
