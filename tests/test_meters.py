"""Meter classes, the group registry and cross-rank merging (optimus_dl/modules/metrics/base.py:30-745,
optimus_dl/modules/metrics/common.py:29-766)."""

import math
import time

import pytest

from optimus_dl_b200.metrics import base as mb
from optimus_dl_b200.metrics import common as mc


def test_average_meter_weights_rounding_and_merge():
    m = mc.AverageMeter(round=2)
    assert m.compute() == 0.0
    m.log(1.0, 1.0)
    m.log(4.0, 3.0)
    assert m.compute() == round(13.0 / 4.0, 2)
    other = mc.AverageMeter()
    other.log(10.0, 4.0)
    m.merge(other.state_dict())
    assert m.compute() == round(53.0 / 8.0, 2)
    clone = mc.AverageMeter()
    clone.load_state_dict(m.state_dict())
    assert clone.compute() == m.compute()


def test_summed_max_min_meters():
    s = mc.SummedMeter()
    for v in (1, 2.5, 3):
        s.log(v)
    assert s.compute() == 6.5
    hi, lo = mc.MaxMeter(), mc.MinMeter()
    assert hi.compute() == -float("inf") and lo.compute() == float("inf")     # nothing logged: the identity elements
    for v in (3, -1, 7):
        hi.log(v)
        lo.log(v)
    assert hi.compute() == 7 and lo.compute() == -1
    other = mc.MaxMeter()
    other.log(11)
    hi.merge(other.state_dict())
    assert hi.compute() == 11
    empty = mc.MinMeter()
    lo.merge(empty.state_dict())                  # a rank that logged nothing does not disturb the result
    assert lo.compute() == -1


def test_exponent_meter_is_exp_of_weighted_mean_and_saturates():
    m = mc.AveragedExponentMeter()
    m.log(1.0, 2.0)
    m.log(2.0, 2.0)
    assert abs(m.compute() - math.exp(1.5)) < 1e-9
    big = mc.AveragedExponentMeter()
    big.log(1e6, 1.0)
    assert big.compute() == float("inf")


def test_stopwatch_and_frequency_meters_measure_milliseconds():
    sw = mc.StopwatchMeter()
    with pytest.raises(AssertionError, match="Stopwatch was never started"):
        sw.end()
    sw.log("end")                                 # as an event, an end whose start was lost (a restart) is dropped
    assert sw.compute() == 0 and sw.counter == 0 and sw._start is None
    sw.log("start")
    time.sleep(0.02)
    sw.log("end")
    assert 15.0 < sw.compute() < 200.0
    with pytest.raises(AssertionError, match="Unknown mode"):
        sw.log("pause")
    known = mc.StopwatchMeter()
    known.elapsed, known.counter = 4_000_000, 2   # nanoseconds over two intervals
    assert known.compute() == 2.0
    fq = mc.FrequencyMeter()
    fq.log()
    assert fq.compute() == 0.0                    # one occurrence: no interval yet
    time.sleep(0.01)
    fq.log()
    assert 5.0 < fq.compute() < 200.0
    restored = mc.FrequencyMeter()
    restored.load_state_dict(fq.state_dict())
    assert restored.start is None and restored.compute() == fq.compute() and fq.counter == 1
    a, b = mc.FrequencyMeter(), mc.FrequencyMeter()
    a.elapsed, a.counter, b.elapsed, b.counter = 1_000_000, 1, 2_000_000, 2
    a.merge(b.state_dict())
    assert (a.elapsed, a.counter, a.compute()) == (3_000_000, 3, 1.0)
    # the minimum is kept as the maximum of the negated values (optimus_dl/modules/metrics/common.py:146-180)
    assert mc.MaxMeter(round=2).value == -float("inf") and mc.MinMeter().value == -float("inf")
    lo = mc.MinMeter()
    lo.log(4.0), lo.log(2.5)
    assert lo.state_dict()["value"] == -2.5 and lo.compute() == 2.5
    ex = mc.AveragedExponentMeter(round=3)
    ex.log(1.0, 2.0)
    assert ex.state_dict() == {"internal": {"round": None, "sum": 2.0, "count": 2.0}, "round": 3}
    older = mc.AveragedExponentMeter.from_state_dict({"sum": 2.0, "count": 2.0, "round": 3})   # the flat form still loads
    assert older.compute() == ex.compute() == 2.718
    assert mc.MaxMeter().compute() == -float("inf")         # nothing logged yet


def test_gather_meter_collects_and_merges():
    g = mc.GatherMeter()
    g.log({"a": 1})
    g.log([2])
    other = mc.GatherMeter()
    other.log("x")
    g.merge(other.state_dict())
    assert g.compute() == [{"a": 1}, [2], "x"]


def test_logging_outside_a_group_is_dropped_and_lazy_values_run_only_on_log_steps():
    mc.log_summed("orphan", 1.0)                  # no active group: nothing is created
    assert mb.get_group("train") is None
    calls = []

    def lazy():
        calls.append(1)
        return 5.0

    for step in range(4):
        with mb.meters_group("train", log_freq=2) as should_log:
            assert should_log == (step % 2 == 0)    # the first step logs, then every second one
            mc.log_averaged("v", lazy)
        mb.step_meters("train")
    assert len(calls) == 2                        # evaluated on the two logging steps only
    assert mb.compute_meters("train")["v"] == 5.0


def test_priority_orders_keys_and_reset_keeps_persistent_meters():
    with mb.meters_group("g", log_freq=1, log_logger_overhead=False):
        mc.log_summed("zeta", 1.0, priority=0)
        mc.log_summed("alpha", 1.0, priority=5)
        mc.log_summed("beta", 1.0, priority=5)
        mc.log_summed("forever", 2.0, reset=False)
    assert list(mb.compute_meters("g")) == ["zeta", "alpha", "beta", "forever"]
    mb.reset_meters("g")
    assert list(mb.compute_meters("g")) == ["forever"]
    with mb.meters_group("g"):
        mc.log_summed("forever", 3.0, reset=False)
    assert mb.compute_meters("g")["forever"] == 5.0


def test_nested_and_sibling_groups_receive_the_same_log_call():
    with mb.meters_group("outer", log_freq=1):
        with mb.meters_group("inner", log_freq=1):
            mc.log_summed("x", 1.0)
        mc.log_summed("x", 10.0)
    assert mb.compute_meters("inner")["x"] == 1.0
    assert mb.compute_meters("outer")["x"] == 11.0


def test_group_state_round_trip_restores_iteration_and_values():
    for _ in range(3):
        with mb.meters_group("train", log_freq=5):
            mc.log_summed("tokens", 4.0, reset=False)
        mb.step_meters("train")
    sd = mb.state_dict()
    mb.clear_all()
    assert mb.compute_meters("train") == {}
    mb.load_state_dict(sd)
    g = mb.get_group("train")
    assert g._iteration == 3 and g.log_freq == 5
    with mb.meters_group("train") as should_log:
        assert not should_log                     # counter 3: not a multiple of 5
    mb.step_meters("train")
    mb.step_meters("train")
    with mb.meters_group("train") as should_log:
        assert should_log                         # counter 5


class _TwoRanks:
    """Collective stand-in whose object all-gather returns this rank's state plus a prepared peer state."""

    world_size = 2

    def __init__(self, peer_states):
        self.peer = peer_states

    def all_gather_objects(self, obj):
        return [obj, self.peer]


def test_aggregation_merges_every_rank_including_keys_only_a_peer_has():
    with mb.meters_group("eval", log_freq=1):
        mc.log_averaged("loss", 2.0, weight=10.0, priority=0)
        mc.log_summed("tokens", 10.0)
    peer_loss, peer_tok, peer_only = mc.AverageMeter(), mc.SummedMeter(), mc.MaxMeter()
    peer_loss.log(4.0, 30.0)
    peer_tok.log(30.0)
    peer_only.log(9.0)
    peer = {"loss": mb.MeterEntry(peer_loss, True, 0).state_dict(), "tokens": mb.MeterEntry(peer_tok, True, 100).state_dict(),
            "peak": mb.MeterEntry(peer_only, True, 100).state_dict()}
    assert "ms_spent_logging" in mb.compute_meters("eval")   # the group accounts for its own logging time
    out = mb.compute_meters("eval", aggregate=True, collective=_TwoRanks(peer))
    assert abs(out["loss"] - 3.5) < 1e-9 and out["tokens"] == 40.0 and out["peak"] == 9.0
    assert list(out)[0] == "loss"
    assert mb.compute_meters("eval")["tokens"] == 10.0       # local values are untouched by aggregation
    # a peer may also send bare meter states; class and priority are then those of the local meter of that name
    bare = {"loss": peer_loss.state_dict(), "tokens": peer_tok.state_dict(), "peak": peer_only.state_dict()}
    out = mb.compute_meters("eval", aggregate=True, collective=_TwoRanks(bare))
    assert abs(out["loss"] - 3.5) < 1e-9 and out["tokens"] == 40.0 and "peak" not in out


def test_entry_and_group_structure():
    """Defaults, state keys and cadence of optimus_dl/modules/metrics/base.py (MeterEntry, MeterGroup)."""
    entry = mb.MeterEntry(meter=mc.AverageMeter())
    assert entry.reset is False and entry.priority == 0
    state = mb.MeterEntry(meter=mc.AverageMeter(), reset=True, priority=10).state_dict()
    assert state["meter_class"] == "AverageMeter" and state["reset"] is True and state["priority"] == 10
    entry.load_state_dict({"meter": {"sum": 10.0, "count": 1.0, "round": None}, "reset": True, "priority": 5,
                           "meter_class": "AverageMeter"})
    assert isinstance(entry.meter, mc.AverageMeter) and entry.meter.compute() == 10.0 and entry.priority == 5
    dotted = mb.MeterEntry.from_state_dict({"meter": {"round": None, "sum": 2.0}, "reset": False, "priority": 1,
                                            "meter_class": "optimus_dl_b200.metrics.common.SummedMeter"})
    assert isinstance(dotted.meter, mc.SummedMeter)

    group = mb.MeterGroup("g", log_freq=3)
    assert mb.MeterGroup("d").log_freq == 1 and group._iteration_counter == 0 and len(group._meters) == 0
    assert group.should_log()                                   # counter 0 is a logging step
    assert not group.step() and not group.should_log()          # 1
    assert not group.step()                                     # 2
    assert group.step() and group.should_log()                  # 3
    group.add_meter("high", mb.MeterEntry(meter=mc.AverageMeter(), priority=10))
    group.add_meter("low", mb.MeterEntry(meter=mc.SummedMeter(), priority=1, reset=True))
    group.add_meter("mid", mb.MeterEntry(meter=mc.AverageMeter(), priority=5))
    assert group._keys_sorted == ["low", "mid", "high"] and group.get_meter("none") is None
    group.reset()
    assert group._keys_sorted == ["mid", "high"]                # only reset=True meters are dropped
