"""Learning-rate schedules against their closed forms (optimus_dl/modules/lr_scheduler/base.py:20-87,
wsd_scheduler.py:14-234, linear_warmup.py:12-90, cosine_annealing.py:14-85)."""

import math

import pytest
import torch

from optimus_dl_b200.lr_scheduler import build_lr_scheduler


def _opt(*lrs):
    groups = [{"params": [torch.nn.Parameter(torch.zeros(1))], "lr": lr} for lr in (lrs or (1.0,))]
    return torch.optim.SGD(groups, lr=1.0)


def _wsd(o, iterations, **kw):
    return build_lr_scheduler({"_name": "wsd", **kw}, optimizer=o, iterations=iterations)


def _at(s, step):
    s._step_count = step
    s.set()
    return s.get_last_lr()


def test_wsd_warmup_starts_at_base_over_div_factor_and_is_linear():
    o = _opt(2.0)
    s = _wsd(o, 1000, warmup_steps=100, init_div_factor=50, fract_decay=0.1)
    assert _at(s, 0) == [pytest.approx(2.0 / 50)]
    assert _at(s, 50) == [pytest.approx(2.0 * (0.5 + 0.5 / 50))]
    assert _at(s, 100) == [2.0]
    assert _at(s, 899) == [2.0]                      # stable phase lasts until the last 10 %
    assert _at(s, 1000) == [0.0] and _at(s, 5000) == [0.0]


def test_wsd_warmup_from_fraction_and_missing_both_is_an_error():
    s = _wsd(_opt(), 200, warmup_steps=None, warmup_steps_fraction=0.25)
    assert s.warmup_steps == 50
    with pytest.raises(AssertionError):
        _wsd(_opt(), 200, warmup_steps=None, warmup_steps_fraction=None)


@pytest.mark.parametrize("kind,f", [
    ("linear", lambda x, lo: lo + (1 - lo) * (1 - x)),
    ("cosine", lambda x, lo: lo + (1 - lo) * (1 + math.cos(math.pi * x)) / 2),
    ("square", lambda x, lo: lo + (1 - lo) * (1 - x * x)),
    ("sqrt", lambda x, lo: lo + (1 - lo) * (1 - math.sqrt(x))),
    ("exp", lambda x, lo: lo ** x),
    ("miror_cosine", lambda x, lo: 2 * (lo + (1 - lo) * (1 - x)) - (lo + (1 - lo) * (1 + math.cos(math.pi * x)) / 2)),
])
def test_wsd_decay_shapes_follow_their_formulas(kind, f):
    lo = 0.1
    o = _opt(3.0)
    s = _wsd(o, 100, warmup_steps=0, fract_decay=0.4, decay_type=kind, final_lr_factor=lo)
    for step in (60, 61, 70, 85, 99):
        x = (step - 60) / 40
        assert _at(s, step) == [pytest.approx(3.0 * f(x, lo), rel=1e-9)], (kind, step)
    assert _at(s, 100) == [pytest.approx(3.0 * lo)]


def test_wsd_piecewise_linear_passes_through_its_waypoints():
    s = _wsd(_opt(), 100, warmup_steps=0, fract_decay=0.3, decay_type="linear_pw", linear_pw_subdivisions=[0.5, 0.2],
             final_lr_factor=0.0)
    # three equal segments over steps 70..100: 1.0 -> 0.5 -> 0.2 -> 0.0
    assert _at(s, 70) == [pytest.approx(1.0)]
    assert _at(s, 80) == [pytest.approx(0.5)]
    assert _at(s, 90) == [pytest.approx(0.2)]
    assert _at(s, 75) == [pytest.approx(0.75)]
    assert _at(s, 95) == [pytest.approx(0.1)]


def test_wsd_cooldown_can_start_below_the_plateau():
    s = _wsd(_opt(), 100, warmup_steps=0, fract_decay=0.5, decay_type="linear", cooldown_start_lr_factor=0.6,
             final_lr_factor=0.2)
    assert _at(s, 49) == [1.0]
    assert _at(s, 50) == [pytest.approx(0.6)] and _at(s, 75) == [pytest.approx(0.4)]


def test_every_parameter_group_keeps_its_own_base_rate():
    o = _opt(1.0, 0.1, 5.0)
    s = _wsd(o, 100, warmup_steps=10, init_div_factor=10, fract_decay=0.2)
    assert _at(s, 5) == [pytest.approx(b * (0.5 + 0.05)) for b in (1.0, 0.1, 5.0)]
    assert _at(s, 90) == [pytest.approx(b * 0.5) for b in (1.0, 0.1, 5.0)]
    o.param_groups.append({"params": [], "lr": 1.0})
    with pytest.raises(ValueError):
        s.set()                                       # a group added behind the schedule's back is reported


def test_step_counts_and_state_round_trip_across_schedule_types():
    for cfg in ({"_name": "wsd", "warmup_steps": 3, "fract_decay": 0.5, "decay_type": "cosine"},
                {"_name": "linear_warmup", "warmup_steps": 4, "start_lr": 0.1},
                {"_name": "cosine_annealing", "eta_min": 0.05}):
        o1 = _opt(1.0, 2.0)
        s1 = build_lr_scheduler(dict(cfg), optimizer=o1, iterations=20)
        for _ in range(9):
            s1.step()
        assert s1.last_epoch == 9 and s1.get_last_lr() == [g["lr"] for g in o1.param_groups]
        o2 = _opt(7.0, 7.0)                             # different starting rates: the state must win
        s2 = build_lr_scheduler(dict(cfg), optimizer=o2, iterations=20)
        s2.load_state_dict(s1.state_dict())
        assert s2.last_epoch == 9 and s2.get_last_lr() == pytest.approx(s1.get_last_lr())
        for _ in range(6):
            s1.step()
            s2.step()
        assert s2.get_last_lr() == pytest.approx(s1.get_last_lr()), cfg["_name"]


def test_linear_warmup_targets_and_zero_length():
    o = _opt(1.0, 4.0)
    s = build_lr_scheduler({"_name": "linear_warmup", "warmup_steps": 10, "start_lr": 0.5, "target_lr": 2.0}, optimizer=o,
                           iterations=100)
    assert _at(s, 0) == [0.5, 0.5] and _at(s, 5) == [pytest.approx(1.25)] * 2 and _at(s, 10) == [2.0, 2.0]
    assert _at(s, 60) == [2.0, 2.0]
    o = _opt(3.0)
    s = build_lr_scheduler({"_name": "linear_warmup", "warmup_steps": 0}, optimizer=o, iterations=10)
    assert _at(s, 0) == [3.0]
    with pytest.raises(ValueError):
        build_lr_scheduler({"_name": "linear_warmup", "warmup_steps": None, "warmup_percent": None}, optimizer=_opt(),
                           iterations=10)


def test_cosine_uses_the_run_length_and_ignores_unread_keys():
    o = _opt(1.0)
    s = build_lr_scheduler({"_name": "cosine_annealing", "eta_min": 0.0, "T_max": 3, "min_lr_ratio": 0.5}, optimizer=o,
                           iterations=40)
    for step in (0, 10, 20, 40):
        assert _at(s, step) == [pytest.approx(0.5 * (1 + math.cos(math.pi * step / 40)), abs=1e-12)]
