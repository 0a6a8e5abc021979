"""``model_info``: static facts about the model (optimus_dl/modules/metrics/sources/model_info.py)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ...core.model_utils import get_num_parameters
from ..source import MetricSource, MetricSourceConfig, StandardProtocols as P, register_metric_source


@dataclass
class ModelInfoSourceConfig(MetricSourceConfig):
    only_trainable: bool = False


@register_metric_source("model_info", ModelInfoSourceConfig)
class ModelInfoSource(MetricSource):
    provides = {P.MODEL_PARAMETERS_COUNT}

    def __call__(self, dependencies: dict[str, Any], model: Any = None, **kwargs: Any):
        return {P.MODEL_PARAMETERS_COUNT: get_num_parameters(model, only_trainable=bool(self.cfg.only_trainable))}
