"""LR schedules, meters, meter groups and the metric engine."""

import math

import pytest
import torch

from optimus_dl_b200.lr_scheduler import build_lr_scheduler
from optimus_dl_b200.metrics import (MetricEngine, compute_meters, log_averaged, log_summed, meters_group, reset_meters,
                                     state_dict, step_meters, load_state_dict)
from optimus_dl_b200.metrics import base as mb


def _opt(lr=1.0):
    return torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=lr)


def _trace(s, o, n):
    out = []
    for _ in range(n):
        out.append(o.param_groups[0]["lr"])
        s.step()
    return out


def test_wsd_shapes_and_state_roundtrip():
    o = _opt()
    s = build_lr_scheduler({"_name": "wsd", "warmup_steps": 10, "fract_decay": 0.2, "decay_type": "linear", "init_div_factor": 100},
                           optimizer=o, iterations=100)
    v = _trace(s, o, 101)
    assert v[0] == pytest.approx(0.01) and v[10] == 1.0 and v[79] == 1.0 and v[90] == pytest.approx(0.5) and v[100] == 0.0
    for kind in ("cosine", "exp", "square", "sqrt", "miror_cosine", "linear_pw"):
        o2 = _opt()
        extra = {"linear_pw_subdivisions": [0.5, 0.1]} if kind == "linear_pw" else {}
        s2 = build_lr_scheduler({"_name": "wsd", "warmup_steps": 0, "fract_decay": 0.5, "decay_type": kind, "final_lr_factor": 0.1, **extra},
                                optimizer=o2, iterations=20)
        w = _trace(s2, o2, 20)
        assert w[0] == 1.0 and w[10] <= 1.0 and all(a >= b - 1e-9 for a, b in zip(w[10:], w[11:])), kind
    with pytest.raises(ValueError):
        build_lr_scheduler({"_name": "wsd", "decay_type": "nope"}, optimizer=_opt(), iterations=10)
    o3 = _opt()
    s3 = build_lr_scheduler({"_name": "wsd", "warmup_steps": 5}, optimizer=o3, iterations=50)
    for _ in range(7):
        s3.step()
    o4 = _opt()
    s4 = build_lr_scheduler({"_name": "wsd", "warmup_steps": 5}, optimizer=o4, iterations=50)
    s4.load_state_dict(s3.state_dict())
    assert o4.param_groups[0]["lr"] == o3.param_groups[0]["lr"] and s4.last_epoch == 7


def test_cosine_and_linear_warmup():
    o = _opt(2.0)
    s = build_lr_scheduler({"_name": "cosine_annealing", "eta_min": 0.2, "T_max": 5, "warmup_percent": 0.1}, optimizer=o, iterations=10)
    v = _trace(s, o, 11)
    assert v[0] == 2.0 and v[5] == pytest.approx(0.2 + 1.8 * 0.5) and v[10] == pytest.approx(0.2)
    o = _opt(1.0)
    s = build_lr_scheduler({"_name": "linear_warmup", "warmup_percent": 0.5, "start_lr": 0.0}, optimizer=o, iterations=10)
    v = _trace(s, o, 8)
    assert v[0] == 0.0 and v[5] == 1.0 and v[7] == 1.0


def test_meter_groups_lazy_values_reset_and_state():
    calls = []
    for it in range(4):
        with meters_group("g", log_freq=2) as should_log:
            assert should_log == (it % 2 == 0)
            log_averaged("loss", lambda: calls.append(it) or float(it), weight=2, round=3)
            log_summed("total", 1.0, reset=False)
        if should_log:
            out = compute_meters("g")
            assert out["loss"] == float(it) and out["total"] == it + 1
            reset_meters("g")
        step_meters("g")
    assert calls == [0, 2]           # lazy values are only evaluated on logging steps
    sd = state_dict()
    mb.clear_all()
    load_state_dict(sd)
    assert compute_meters("g")["total"] == 4


def test_metric_engine_protocols_sources_and_caching():
    from optimus_dl_b200.metrics.source import MetricSource, register_metric_source

    counter = {"n": 0}

    class _Src(MetricSource):
        provides = {"loss"}

        def __call__(self, dependencies, **kw):
            counter["n"] += 1
            return {"loss": torch.tensor(2.0)}

    try:
        register_metric_source("test_const_loss")(_Src)
    except AssertionError:
        pass
    cfgs = [{"_name": "source_group", "prefix": "a", "sources": {"s": {"_name": "test_const_loss"}}, "metrics": [{"_name": "loss"}]},
            {"_name": "source_group", "prefix": "b", "sources": {"s": {"_name": "test_const_loss"}}, "metrics": [{"_name": "loss"}]},
            {"_name": "accuracy"}]
    e = MetricEngine("eng", cfgs)
    assert e.required_external_protocols == {"classification"}
    pred = torch.tensor([[1, 2, 3]])
    e.update({}, {"classification": {"predictions": pred, "targets": torch.tensor([[1, 0, 3]]), "mask": torch.ones(1, 3, dtype=torch.bool)}})
    assert counter["n"] == 1        # identical sources are evaluated once per batch across groups
    out = e.compute(compute_meters("eng"))
    assert out["a/loss_metric/loss"] == 2.0 and out["b/loss_metric/loss"] == 2.0
    assert out["accuracy_metric/accuracy"] == pytest.approx(2 / 3)
