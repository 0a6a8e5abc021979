"""MetricEngine: source hashing and caching, dependency resolution, cycles, missing protocols, failure isolation,
custom metrics with internal sub-metrics and finalisers (optimus_dl/modules/metrics/engine.py,
metrics/source.py:20-106, metrics/metrics.py:22-207)."""

import math
from dataclasses import dataclass, field

import pytest
import torch

from optimus_dl_b200.metrics import base as mb
from optimus_dl_b200.metrics.engine import MetricEngine
from optimus_dl_b200.metrics.metrics import Metric, MetricConfig, register_metric
from optimus_dl_b200.metrics.source import MetricSource, MetricSourceConfig, register_metric_source

CALLS: dict = {}


@dataclass
class _ConstCfg(MetricSourceConfig):
    value: float = 1.0
    provide: str = "loss"
    need: list = field(default_factory=list)
    fail: bool = False


class _Const(MetricSource):
    @property
    def provides(self):
        return {self.cfg.provide}

    @property
    def requires(self):
        return set(self.cfg.need)

    def __call__(self, dependencies, **kw):
        CALLS[self.cfg.provide] = CALLS.get(self.cfg.provide, 0) + 1
        if self.cfg.fail:
            raise RuntimeError("source failed")
        extra = sum(float(v) for v in dependencies.values())
        return {self.cfg.provide: torch.tensor(float(self.cfg.value) + extra)}


class _Ratio(Metric):
    """Two internal sums and a finaliser that divides them (the internal keys disappear from the result)."""

    requires = {"loss"}
    accumulators = {"_num": "sum", "_den": "sum"}

    def __call__(self, data):
        return {"_num": {"value": float(data["loss"])}, "_den": {"value": 2.0}}

    def finalize(self, agg):           # this metric's own accumulators, keyed by sub-metric name
        return {"ratio": agg["_num"] / agg["_den"]}


def _register():
    for name, cls, cfg, reg in (("t_const", _Const, _ConstCfg, register_metric_source),):
        try:
            reg(name, cfg)(cls)
        except (AssertionError, ValueError, KeyError):
            pass
    try:
        register_metric("t_ratio", MetricConfig)(_Ratio)
    except (AssertionError, ValueError, KeyError):
        pass


@pytest.fixture(autouse=True)
def _fresh():
    _register()
    CALLS.clear()
    yield


def _src(**kw):
    return {"_name": "t_const", **kw}


def test_equal_configs_share_one_evaluation_and_different_configs_do_not():
    e = MetricEngine("g", [
        {"_name": "source_group", "prefix": "a", "sources": {"s": _src(value=2.0)}, "metrics": [{"_name": "loss"}]},
        {"_name": "source_group", "prefix": "b", "sources": {"other_role": _src(value=2.0)}, "metrics": [{"_name": "loss"}]},
        {"_name": "source_group", "prefix": "c", "sources": {"s": _src(value=5.0)}, "metrics": [{"_name": "loss"}]},
    ])
    assert e.required_external_protocols == set()
    e.update({})
    assert CALLS["loss"] == 2                       # value 2.0 once (shared by a and b), value 5.0 once
    out = e.compute(mb.compute_meters("g"))
    assert out["a/loss_metric/loss"] == 2.0 and out["b/loss_metric/loss"] == 2.0 and out["c/loss_metric/loss"] == 5.0
    e.update({})                                    # the cache lives for one batch only
    assert CALLS["loss"] == 4
    hashes = {g.sources[r].config_hash for g in e.groups for r in g.sources}
    assert len(hashes) == 2


def test_sources_may_depend_on_other_sources_of_their_group():
    e = MetricEngine("g", [{"_name": "source_group", "prefix": "", "sources": {
        "base": _src(value=3.0, provide="hidden"),
        "top": _src(value=1.0, provide="loss", need=["hidden"]),
    }, "metrics": [{"_name": "loss"}]}])
    e.update({})
    assert e.compute(mb.compute_meters("g"))["loss_metric/loss"] == 4.0 and CALLS == {"hidden": 1, "loss": 1}


def test_cycles_and_missing_protocols_are_reported_without_stopping_other_metrics(caplog):
    e = MetricEngine("g", [
        {"_name": "source_group", "prefix": "cyc", "sources": {
            "x": _src(provide="loss", need=["hidden"]), "y": _src(provide="hidden", need=["loss"])},
         "metrics": [{"_name": "loss"}]},
        {"_name": "source_group", "prefix": "miss", "sources": {"x": _src(provide="loss", need=["nowhere"])},
         "metrics": [{"_name": "loss"}]},
        {"_name": "source_group", "prefix": "bad", "sources": {"x": _src(fail=True, value=9.0)},
         "metrics": [{"_name": "loss"}, {"_name": "loss", "nested_name": "again"}]},
        {"_name": "source_group", "prefix": "ok", "sources": {"x": _src(value=7.0)}, "metrics": [{"_name": "loss"}]},
    ])
    with caplog.at_level("ERROR"):
        e.update({})
    out = e.compute(mb.compute_meters("g"))
    assert out == {k: v for k, v in out.items() if k.startswith("ok/") or k == "ms_spent_logging"} and out["ok/loss_metric/loss"] == 7.0
    text = caplog.text
    assert "Cyclic dependency" in text and "nowhere" in text and "source failed" in text
    assert CALLS.get("loss", 0) == 2                # the failing source ran once; its error was cached for the second metric


def test_external_protocols_are_taken_from_the_criterion_and_override_sources():
    e = MetricEngine("g", [{"_name": "perplexity"}, {"_name": "accuracy"},
                           {"_name": "source_group", "prefix": "s", "sources": {"x": _src(value=1.0)}, "metrics": [{"_name": "loss"}]}])
    assert e.required_external_protocols == {"loss", "classification"}
    logits = torch.tensor([[[2.0, 0.0, 0.0], [0.0, 3.0, 0.0]]])
    targets = torch.tensor([[0, 2]])
    nll = torch.nn.functional.cross_entropy(logits[0], targets[0])
    given = {"logits": logits, "logits_targets": targets, "loss": nll,
             "classification": {"predictions": logits.argmax(-1), "targets": targets, "mask": targets != -100}}
    e.update({}, given)
    out = e.compute(mb.compute_meters("g"))
    assert out["perplexity_metric/perplexity"] == pytest.approx(math.exp(nll.item()), rel=1e-5)
    assert out["accuracy_metric/accuracy"] == 0.5        # named as optimus_dl/modules/metrics/engine.py:306-318 names it
    assert out["accuracy_metric/total"] == 2            # the count of valid positions, summed over batches
    assert out["s/loss_metric/loss"] == pytest.approx(nll.item()) and "loss" not in CALLS      # a value the caller already has is not recomputed


def test_nested_names_internal_submetrics_and_finalisers():
    e = MetricEngine("g", [{"_name": "source_group", "prefix": "p", "sources": {"x": _src(value=6.0)},
                            "metrics": [{"_name": "t_ratio", "nested_name": "r"}, {"_name": "loss"}]}])
    e.update({})
    e.update({})
    raw = mb.compute_meters("g")
    assert raw["_internal/p/r/_num"] == 12.0 and raw["_internal/p/r/_den"] == 4.0
    out = e.compute(raw)
    assert out["p/r/ratio"] == 3.0 and out["p/loss_metric/loss"] == 6.0
    assert not [k for k in out if k.startswith("_internal/")]


def test_updates_outside_logging_steps_cost_nothing():
    e = MetricEngine("g", [{"_name": "source_group", "prefix": "", "sources": {"x": _src(value=1.0)}, "metrics": [{"_name": "loss"}]}])
    for step in range(4):
        with mb.meters_group("g", log_freq=4):
            e.update({})
        mb.step_meters("g")
    assert CALLS["loss"] == 1                        # only the fourth step is a logging step


def test_config_errors():
    with pytest.raises(ValueError):
        MetricEngine("g", [{"_name": "source_group", "sources": {}}])          # no metrics key
    assert MetricEngine("g", []).required_external_protocols == set()
    assert MetricEngine("g", None).compute({"a": 1}) == {"a": 1}
    two = MetricEngine("g", [{"_name": "source_group", "sources": {"x": _src()}, "metrics": [{"_name": "loss"}]},
                             {"_name": "source_group", "sources": {"x": _src()}, "metrics": [{"_name": "loss"}]}])
    assert [g.prefix for g in two.groups] == ["group_0", "group_1"]            # default prefixes keep groups apart
