"""Config tree, registry validation, lazy instantiation and composition (behaviour specs follow the
reference's tests/core/*)."""

import os
import textwrap
from dataclasses import dataclass, field

import pytest

from optimus_dl_b200.core import compose, conf
from optimus_dl_b200.core.config_utils import non_resolving_instantiate as nri
from optimus_dl_b200.core.registry import (ConfigValidationError, RegistryConfig, RegistryConfigStrict, make_registry,
                                           validate_and_cast)


def test_interpolation_absolute_relative_nested_and_templates():
    c = conf.create({"a": {"b": 3, "c": "${.b}", "d": "${..x}", "e": "v-${a.b}-${x}"}, "x": 7, "k": "b", "n": "${a.${k}}"})
    assert c.a.c == 3 and c.a.d == 7 and c.a.e == "v-3-7" and c.n == 3
    c.a.b = 5
    assert c.a.c == 5 and c.n == 5
    with pytest.raises(conf.MissingMandatoryValue):
        conf.create({"m": "???"}).m
    with pytest.raises(conf.InterpolationError):
        conf.create({"p": "${q}", "q": "${p}"}).p


def test_resolvers_env_eval_hash():
    os.environ["OB_TEST_ENV"] = "hello"
    c = conf.create({"a": "${oc.env:OB_TEST_ENV}", "b": "${oc.env:OB_MISSING,fallback}", "c": "${eval:'2 ** 5'}",
                     "h": "${config_hash:}", "cpu": "${cpu_count:}"})
    nri(c)
    assert c.a == "hello" and c.b == "fallback" and c.c == 32
    assert len(c.h) == 16 and c.cpu >= 1


def test_merge_update_select_to_container():
    a = conf.create({"x": {"y": 1, "z": [1, 2]}, "k": "${x.y}"})
    m = conf.merge(a, {"x": {"y": 2, "w": 3}})
    assert conf.to_container(m, resolve=True) == {"x": {"y": 2, "z": [1, 2], "w": 3}, "k": 2}
    conf.update(m, "x.new.deep", 4)
    assert conf.select(m, "x.new.deep") == 4 and conf.select(m, "nope.q", default=9) == 9
    assert conf.to_container(a, resolve=False)["k"] == "${x.y}"


def test_lazy_targets_react_to_changes_and_detect_cycles():
    c = nri({"p": {"v": 10.5}, "a": {"_target_": "math.ceil", "_args_": ["${p.v}"]}, "ref": "${a}",
             "lst": [{"_target_": "math.floor", "_args_": [3.2]}, "${..p.v}"]})
    assert c.a == 11 and c.ref == 11 and c.lst[0] == 3 and c.lst[1] == 10.5
    c.p.v = 20.1
    assert c.a == 21 and c.ref == 21
    cyc = nri({"a": {"_target_": "builtins.dict", "x": "${b}"}, "b": {"_target_": "builtins.dict", "y": "${a}"}})
    with pytest.raises(conf.InterpolationError):
        cyc.a
    eager = nri({"o": {"_target_": "builtins.dict", "k": 1}}, lazy=False)
    assert eager.o.k == 1


@dataclass
class _Inner:
    n: int = 1
    tags: list[str] = field(default_factory=list)


@dataclass
class _StrictCfg(RegistryConfigStrict):
    lr: float = 1e-3
    betas: tuple[float, float] = (0.9, 0.999)
    inner: _Inner = field(default_factory=_Inner)
    opt: int | None = None
    mode: str | int = "a"


@dataclass
class _FlexCfg(RegistryConfig):
    a: int = 1


def test_registry_strict_flexible_and_casting():
    reg, register, build = make_registry("test_reg_a")

    @register("thing", _StrictCfg)
    class Thing:
        def __init__(self, cfg, extra=None):
            self.cfg, self.extra = cfg, extra

    t = build({"_name": "thing", "lr": "3e-4", "inner": {"n": "4"}, "opt": None, "mode": 3}, extra=5)
    assert t.cfg.lr == pytest.approx(3e-4) and t.cfg.inner.n == 4 and t.cfg.betas == [0.9, 0.999] and t.cfg.mode == "3"   # first castable member of str | int
    assert t.extra == 5 and build("thing").cfg.lr == 1e-3
    with pytest.raises(ConfigValidationError):
        build({"_name": "thing", "unknown": 1})
    with pytest.raises(ConfigValidationError):
        build({"_name": "thing", "lr": "fast"})
    with pytest.raises(KeyError):
        build({"_name": "other"})

    @register("flex", _FlexCfg)
    class Flex:
        def __init__(self, cfg):
            self.cfg = cfg

    assert build({"_name": "flex", "whatever": [1, 2]}).cfg.whatever == [1, 2]

    @Thing.register_arch("big")
    def big():
        return _StrictCfg(lr=0.5)

    assert build("thing-big").cfg.lr == 0.5 and build({"_name": "thing-big", "lr": 0.1}).cfg.lr == 0.1
    assert validate_and_cast(int | None, None) is None and validate_and_cast(list[int], ["1", 2]) == [1, 2]


def test_compose_defaults_groups_overrides(tmp_path):
    (tmp_path / "model").mkdir()
    (tmp_path / "opt" / "amp").mkdir(parents=True)
    (tmp_path / "base.yaml").write_text("hydra:\n  job:\n    env_set:\n      OB_COMPOSE_ENV: 1\nshared: 1\n")
    (tmp_path / "model" / "small.yaml").write_text("n: 2\nseq: ${args.seq}\n")
    (tmp_path / "model" / "big.yaml").write_text("n: 48\nseq: ${args.seq}\n")
    (tmp_path / "opt" / "amp" / "bf16.yaml").write_text("dtype: bfloat16\n")
    (tmp_path / "loggers").mkdir()
    (tmp_path / "loggers" / "basic.yaml").write_text("- _name: jsonl\n")
    (tmp_path / "root.yaml").write_text(textwrap.dedent("""
        defaults:
          - base.yaml
          - model: small
          - opt/amp: bf16
          - loggers: basic
          - _self_
        args: {seq: 128}
        model: {extra: true}
        x: {y: 1}
    """))
    c = compose.compose(str(tmp_path), "root")
    assert c.model.n == 2 and c.model.extra is True and c.model.seq == 128 and c.opt.amp.dtype == "bfloat16"
    assert "hydra" not in c and c.shared == 1 and c.loggers[0]._name == "jsonl" and os.environ["OB_COMPOSE_ENV"] == "1"
    c = compose.compose(str(tmp_path), "root", ["model=big", "x.y=5", "+x.z=[1,2]", "++q.r=s", "~shared"])
    assert c.model.n == 48 and c.x.y == 5 and c.x.z == [1, 2] and c.q.r == "s" and "shared" not in c
    assert compose.expand_sweeps(["a=1,2", "b=x"]) == [["a=1", "b=x"], ["a=2", "b=x"]]
    cli = compose.parse_cli(["--config-name=foo", "-m", "a=1", "-cp", "dir"])
    assert cli["config_name"] == "foo" and cli["multirun"] and cli["overrides"] == ["a=1"] and cli["config_path"] == "dir"
