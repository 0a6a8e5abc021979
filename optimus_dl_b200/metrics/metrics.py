"""Stateless metrics and the ``metric`` registry (optimus_dl/modules/metrics/metrics.py:22-207).

A metric names the protocols it ``requires``, returns per-batch ``{sub_metric: log kwargs}`` and
says which accumulator each sub-metric uses (``average | mean | sum | gather | perplexity | max |
min``); ``finalize`` may post-process the aggregated numbers."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F

from ..core.registry import RegistryConfig, make_registry
from .source import StandardProtocols as P


@dataclass
class MetricConfig(RegistryConfig):
    nested_name: str | None = None


class Metric:
    def __init__(self, cfg: Any = None, **kwargs: Any):
        self.cfg = cfg
        self.nested_name = cfg.get("nested_name") if cfg is not None and hasattr(cfg, "get") else None

    @property
    def requires(self) -> set[str]:
        return set()

    @property
    def accumulators(self) -> dict[str, str]:
        return {}

    def __call__(self, sources_data: dict[str, Any]) -> dict[str, dict[str, Any]]:
        raise NotImplementedError

    def finalize(self, aggregated: dict[str, Any]) -> dict[str, Any]:
        """Final values from this metric's aggregated accumulators (sub-metric name -> value); names starting with
        ``_`` are internal and not reported (optimus_dl/modules/metrics/metrics.py:79-89)."""
        return {k: v for k, v in aggregated.items() if not str(k).startswith("_")}


metric_registry, register_metric, build_metric = make_registry("metric", Metric)


@register_metric("accuracy", MetricConfig)
class AccuracyMetric(Metric):
    requires = {P.CLASSIFICATION}
    accumulators = {"accuracy": "average"}

    def __call__(self, sources_data):
        c = sources_data[P.CLASSIFICATION]
        mask = c.get("mask")
        hit = (c["predictions"] == c["targets"])
        if mask is not None:
            n = mask.sum().item()
            return {"accuracy": {"value": (hit & mask).sum().item() / max(n, 1), "weight": n}}
        return {"accuracy": {"value": hit.float().mean().item(), "weight": hit.numel()}}


@register_metric("perplexity", MetricConfig)
class PerplexityMetric(Metric):
    requires = {P.LOGITS, P.LOGITS_TARGETS}
    accumulators = {"perplexity": "perplexity"}

    def __call__(self, sources_data):
        logits, targets = sources_data[P.LOGITS], sources_data[P.LOGITS_TARGETS]
        nll = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), targets.reshape(-1), ignore_index=-100,
                              reduction="sum")
        n = (targets != -100).sum().item()
        return {"perplexity": {"value": nll.item() / max(n, 1), "weight": n}}


@register_metric("loss", MetricConfig)
class LossMetric(Metric):
    requires = {P.LOSS}
    accumulators = {"loss": "average"}

    def __call__(self, sources_data):
        loss = sources_data[P.LOSS]
        return {"loss": {"value": loss.item() if isinstance(loss, torch.Tensor) else float(loss), "weight": 1.0}}


# per-metric config names of the reference (all carry the same fields here)
AccuracyMetricConfig = PerplexityMetricConfig = LossMetricConfig = MetricConfig
