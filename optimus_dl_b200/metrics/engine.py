"""Config-driven metric evaluation (optimus_dl/modules/metrics/engine.py:53-404).

``MetricEngine(group_name, configs)`` takes a list of metric configs, or ``source_group`` entries
``{prefix, sources: {role: cfg}, metrics: [...]}``. Per batch, ``update(data, computed_data)`` feeds
every metric with the protocols it requires: from ``computed_data`` (what the criterion already
produced), else from the group's sources, each evaluated at most once per batch across all groups
(cache keyed by the source's config hash; failures are cached too). Sources may depend on other
sources; cycles are reported. Results go to the meter group ``group_name`` with the accumulator
each metric asks for; ``compute(raw)`` lets metrics post-process the aggregated values."""

from __future__ import annotations

import logging
from typing import Any, Callable

from .base import BaseMeter, log_meter, meters_group
from .common import AverageMeter, AveragedExponentMeter, GatherMeter, MaxMeter, MinMeter, SummedMeter
from .metrics import Metric, build_metric
from .source import MetricSource, build_metric_source

logger = logging.getLogger(__name__)

ACCUMULATORS: dict[str, Callable[[], BaseMeter]] = {
    "average": AverageMeter, "mean": AverageMeter, "sum": SummedMeter, "gather": GatherMeter,
    "perplexity": AveragedExponentMeter, "max": MaxMeter, "min": MinMeter,
}


class ParsedGroup:
    def __init__(self, prefix: str):
        self.prefix = prefix
        self.sources: dict[str, MetricSource] = {}
        self.metrics: list[Metric] = []

    @property
    def protocols_to_sources(self) -> dict[str, list[str]]:
        out: dict[str, list[str]] = {}
        for name, s in self.sources.items():
            for proto in s.provides:
                out.setdefault(proto, []).append(name)
        return out


class MetricEngine:
    def __init__(self, group_name: str, configs: list[Any]):
        self.group_name = group_name
        self.groups: list[ParsedGroup] = []
        configs = list(configs or [])
        for idx, cfg in enumerate(configs):
            if cfg.get("_name") == "source_group":
                prefix = cfg.get("prefix")
                if prefix is None:
                    prefix = f"group_{idx}" if len(configs) > 1 else ""
                if "metrics" not in cfg:
                    raise ValueError(f"source_group config at index {idx} is missing required 'metrics' key")
                sources, metrics = cfg.get("sources", {}) or {}, cfg["metrics"]
            else:
                prefix, sources, metrics = "", {}, [cfg]
            g = ParsedGroup(prefix)
            for role, scfg in sources.items():
                g.sources[role] = build_metric_source(scfg)
            for m in metrics:
                g.metrics.append(build_metric(m))
            self.groups.append(g)

    @property
    def required_external_protocols(self) -> set[str]:
        ext: set[str] = set()
        for g in self.groups:
            internal = set().union(*[s.provides for s in g.sources.values()]) if g.sources else set()
            for m in g.metrics:
                ext |= set(m.requires) - internal
        return ext

    def _eval_source(self, g: ParsedGroup, name: str, data: dict[str, Any], cache: dict[str, Any],
                     evaluating: set[str] | None = None) -> dict[str, Any]:
        src = g.sources[name]
        h = src.config_hash
        if h in cache:
            if isinstance(cache[h], Exception):
                raise cache[h]
            return cache[h]
        evaluating = evaluating if evaluating is not None else set()
        if name in evaluating:
            raise RuntimeError(f"Cyclic dependency detected for source '{name}' in group '{g.prefix}'")
        evaluating.add(name)
        try:
            deps: dict[str, Any] = {}
            try:
                for proto in src.requires:
                    providers = g.protocols_to_sources.get(proto, [])
                    if not providers:
                        raise ValueError(f"No source provides the required protocol {proto}")
                    deps[proto] = self._eval_source(g, providers[0], data, cache, evaluating)[proto]
                result = src(deps, **data)
            except Exception as e:
                cache[h] = e
                raise
            cache[h] = result
            return result
        finally:
            evaluating.discard(name)

    def update(self, data: dict[str, Any], computed_data: dict[str, Any] | None = None) -> None:
        with meters_group(self.group_name) as should_log:
            if not should_log:
                return
            cache: dict[str, Any] = {}
            computed = computed_data or {}
            for g in self.groups:
                for i, metric in enumerate(g.metrics):
                    mname = metric.nested_name or (str(metric.cfg.get("_name", i)) + "_metric")
                    inputs: dict[str, Any] = {}
                    try:
                        for proto in metric.requires:
                            if proto in computed:
                                inputs[proto] = computed[proto]
                                continue
                            providers = g.protocols_to_sources.get(proto, [])
                            if not providers:
                                raise ValueError(f"No source provides the required protocol {proto}")
                            inputs[proto] = self._eval_source(g, providers[0], data, cache)[proto]
                        results = metric(inputs)
                    except Exception as e:
                        logger.exception("metric '%s' in group '%s' failed: %s", mname, g.prefix, e)
                        continue
                    for sub, kwargs in results.items():
                        full = self._full_name(g.prefix, mname, sub)
                        acc = metric.accumulators.get(sub)
                        if acc is None:
                            logger.warning("no accumulator for sub-metric '%s' of '%s'; skipped", sub, mname)
                            continue
                        if acc not in ACCUMULATORS:
                            raise ValueError(f"Unknown accumulator type: {acc}")
                        log_meter(full, ACCUMULATORS[acc], **kwargs)

    @staticmethod
    def _full_name(prefix: str, metric_name: str, sub: str) -> str:
        """``[_internal/][prefix/]metric_name/sub`` (just ``metric_name`` when the two are equal), the naming of
        optimus_dl/modules/metrics/engine.py:306-318: ``accuracy`` of the ``accuracy`` metric is logged as
        ``accuracy_metric/accuracy``; sub-metrics whose name starts with ``_`` are internal."""
        base = f"{metric_name}/{sub}" if metric_name != sub else metric_name
        full = f"{prefix}/{base}" if prefix else base
        return f"_internal/{full}" if sub.startswith("_") else full

    def compute(self, raw_results: dict[str, Any]) -> dict[str, Any]:
        """Finalisation as in optimus_dl/modules/metrics/engine.py:350-404: every metric gets the aggregated values
        of ITS accumulators keyed by sub-metric name (taken out of ``raw_results``), and what its ``finalize`` returns
        is reported under the metric's names again; keys starting with ``_`` are dropped. Consumed entries leave
        ``raw_results`` (the caller's dict), as there."""
        report: dict[str, Any] = {}
        for g in self.groups:
            for i, metric in enumerate(g.metrics):
                mname = metric.nested_name or (str(metric.cfg.get("_name", i)) + "_metric")
                acc_data: dict[str, Any] = {}
                for sub in metric.accumulators:
                    full = self._full_name(g.prefix, mname, sub)
                    if full in raw_results:
                        acc_data[sub] = raw_results.pop(full)
                if not acc_data:
                    continue
                try:
                    finalized = metric.finalize(acc_data)
                except Exception as e:
                    logger.exception("finalize of metric '%s' in group '%s' failed: %s", mname, g.prefix, e)
                    continue
                for k, v in finalized.items():
                    if not str(k).startswith("_"):
                        report[self._full_name(g.prefix, mname, k)] = v
        return raw_results | report
