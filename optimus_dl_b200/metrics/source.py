"""Metric sources: producers of the data metrics consume (optimus_dl/modules/metrics/source.py:20-106).
A source declares the protocols it ``provides`` and ``requires``; its ``config_hash`` lets the engine
evaluate identical sources once per batch even when several groups list them."""

from __future__ import annotations

import hashlib
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any

from ..core import conf
from ..core.registry import RegistryConfigStrict, make_registry


class StandardProtocols:
    MODEL_PARAMETERS_COUNT = "model_parameters_count"
    LOGITS = "logits"
    LOGITS_TARGETS = "logits_targets"
    LOGITS_MASK = "logits_mask"
    INPUT_TOKENS = "input_tokens"
    LOSS = "loss"
    GENERATED_TOKENS = "generated_tokens"
    CLASSIFICATION = "classification"


@dataclass
class MetricSourceConfig(RegistryConfigStrict):
    dependencies: dict[str, str] = field(default_factory=dict)


def _hashable(obj: Any) -> Any:
    if isinstance(obj, (list, tuple)):
        return tuple(_hashable(e) for e in obj)
    if isinstance(obj, dict):
        return tuple(sorted((str(k), _hashable(v)) for k, v in obj.items()))
    return obj


class MetricSource(ABC):
    def __init__(self, cfg: Any, **kwargs: Any):
        self.cfg = cfg
        self._hash: str | None = None

    @property
    def config_hash(self) -> str:
        if self._hash is None:
            plain = conf.to_container(self.cfg, resolve=True) if conf.is_config(self.cfg) else self.cfg
            self._hash = hashlib.md5(f"{type(self).__name__}:{_hashable(plain)}".encode()).hexdigest()
        return self._hash

    @property
    @abstractmethod
    def provides(self) -> set[str]: ...

    @property
    def requires(self) -> set[str]:
        return set()

    @abstractmethod
    def __call__(self, dependencies: dict[str, Any], **kwargs: Any) -> dict[str, Any]: ...


metric_source_registry, register_metric_source, build_metric_source = make_registry("metric_source", MetricSource)
