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
        """Accumulator per sub-metric; by default one averaged sub-metric named like the metric
        (optimus_dl/modules/metrics/metrics.py:54-61)."""
        name = self.cfg.get("_name") if self.cfg is not None and hasattr(self.cfg, "get") else None
        return {str(name): "average"} if name else {}

    def __call__(self, sources_data: dict[str, Any]) -> dict[str, dict[str, Any]]:
        raise NotImplementedError

    def finalize(self, aggregated: dict[str, Any]) -> dict[str, Any]:
        """Final values from this metric's aggregated accumulators (sub-metric name -> value); names starting with
        ``_`` are internal and not reported (optimus_dl/modules/metrics/metrics.py:79-89)."""
        return {k: v for k, v in aggregated.items() if not str(k).startswith("_")}


metric_registry, register_metric, build_metric = make_registry("metric", Metric)


def _mask_weight(sources_data: dict[str, Any]) -> float:
    """Number of valid tokens when the classification view comes along, else 1."""
    c = sources_data.get(P.CLASSIFICATION)
    if c and "mask" in c:
        return c["mask"].sum().item()
    return 1.0


@register_metric("accuracy", MetricConfig)
class AccuracyMetric(Metric):
    """Token accuracy over the valid positions, and their count (``total``, summed)."""

    requires = {P.CLASSIFICATION}
    accumulators = {"accuracy": "average", "total": "sum"}

    def __call__(self, sources_data):
        c = sources_data.get(P.CLASSIFICATION)
        if not c:
            return {}
        mask = c.get("mask")
        hit = (c["predictions"] == c["targets"])
        if mask is not None:
            hit, total = hit & mask, mask.sum().item()
        else:
            total = c["targets"].numel()
        if total == 0:
            return {}
        return {"accuracy": {"value": hit.sum().item() / total, "weight": total}, "total": {"value": total}}


@register_metric("perplexity", MetricConfig)
class PerplexityMetric(Metric):
    """``exp`` of the mean loss. Needs only the LOSS protocol, which the criterion exposes with or without a fused
    head (optimus_dl/modules/metrics/metrics.py:139-168): no logits are materialised for it."""

    requires = {P.LOSS}
    accumulators = {"perplexity": "perplexity"}

    def __call__(self, sources_data):
        loss = sources_data.get(P.LOSS)
        if loss is None:
            return {}
        return {"perplexity": {"value": loss.item() if hasattr(loss, "item") else loss,
                               "weight": _mask_weight(sources_data)}}


@register_metric("loss", MetricConfig)
class LossMetric(Metric):
    requires = {P.LOSS}
    accumulators = {"loss": "average"}

    def __call__(self, sources_data):
        loss = sources_data.get(P.LOSS)
        if loss is None:
            return {}
        return {"loss": {"value": loss.item() if hasattr(loss, "item") else loss, "weight": _mask_weight(sources_data)}}


# per-metric config names of the reference (all carry the same fields here)
AccuracyMetricConfig = PerplexityMetricConfig = LossMetricConfig = MetricConfig
