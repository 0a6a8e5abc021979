"""The typed caster behind strict configs and the registry's build paths
(optimus_dl/core/registry.py:96-257, 283-606), case by case."""

import enum
from dataclasses import dataclass, field
from typing import Any, Literal

import pytest

from optimus_dl_b200.core.registry import (ConfigValidationError, RegistryConfig, RegistryConfigStrict, build, make_registry,
                                           validate_and_cast)


class Color(enum.Enum):
    RED = "red"
    BLUE = "blue"


@dataclass
class Inner:
    n: int = 1
    name: str = "x"


@dataclass
class Strict(RegistryConfigStrict):
    lr: float = 1e-3
    steps: int | None = None
    flag: bool = False
    tags: list[str] = field(default_factory=list)
    pair: tuple[float, float] = (0.9, 0.999)
    inner: Inner = field(default_factory=Inner)
    table: dict[str, int] = field(default_factory=dict)
    color: Color = Color.RED
    mode: Literal["a", "b"] = "a"
    either: int | str = 0
    anything: Any = None


@dataclass
class Flexible(RegistryConfig):
    lr: float = 1e-3


@pytest.mark.parametrize("tp,value,want", [
    (int, "7", 7), (int, 7.0, 7), (float, 3, 3.0), (float, "1e-3", 1e-3), (str, 5, "5"), (str, True, "True"),
    (bool, "yes", True), (bool, "off", False), (bool, 1, True), (bool, 0, False),
    (int | None, None, None), (int | None, "4", 4), (float | str, "fast", "fast"), (int | str, 3, 3), (int | str, "3", 3), (str | int, 3, "3"),
    (list[int], ("1", 2.0), [1, 2]), (list, [1, "a"], [1, "a"]), (tuple[float, float], [1, "2"], [1.0, 2.0]),
    (tuple[int, ...], ["1", 2, 3.0], [1, 2, 3]), (dict[str, float], {"a": "1.5"}, {"a": 1.5}),
    (Color, "blue", Color.BLUE), (Color, "RED", Color.RED), (Color, Color.BLUE, Color.BLUE),
    (Literal["a", "b"], "b", "b"), (Any, object, object),
    (float, "${optimization.lr}", "${optimization.lr}"), (int, "???", "???"),        # interpolations and MISSING pass through
])
def test_values_are_cast_where_it_is_safe(tp, value, want):
    assert validate_and_cast(tp, value) == want


@pytest.mark.parametrize("tp,value", [
    (int, "seven"), (int, 7.5), (int, True), (float, "fast"), (float, False), (bool, "maybe"), (bool, 2), (str, [1]),
    (int, None), (list[int], "12"), (list[int], [1, "x"]), (tuple[float, float], [1.0]), (dict[str, int], [("a", 1)]),
    (dict[str, int], {"a": "one"}), (Color, "green"), (Literal["a", "b"], "c"), (int | None, "x"), (Inner, 5),
])
def test_wrong_values_are_rejected_with_the_path(tp, value):
    with pytest.raises(ConfigValidationError) as err:
        validate_and_cast(tp, value, path="cfg.key")
    assert "cfg.key" in str(err.value)


def test_nested_dataclasses_merge_defaults_and_reject_unknown_keys():
    out = validate_and_cast(Strict, {"lr": "0.5", "inner": {"n": "3"}, "tags": ["a", 1], "table": {"k": "2"}, "color": "blue",
                                     "pair": [0.8, "0.95"], "steps": "10", "either": "word"})
    assert out["lr"] == 0.5 and out["inner"] == {"n": 3, "name": "x"} and out["tags"] == ["a", "1"] and out["table"] == {"k": 2}
    assert out["color"] is Color.BLUE and out["pair"] == [0.8, 0.95] and out["steps"] == 10 and out["either"] == "word"
    assert out["flag"] is False and out["mode"] == "a"                      # untouched fields keep their defaults
    assert validate_and_cast(Strict, Strict(lr=2.0))["lr"] == 2.0           # a dataclass instance is accepted as a mapping
    for bad, where in (({"inner": {"m": 1}}, "inner.m"), ({"nope": 1}, "nope"), ({"inner": 3}, "inner"), ({"mode": "z"}, "mode")):
        with pytest.raises(ConfigValidationError) as err:
            validate_and_cast(Strict, bad)
        assert where in str(err.value)
    flex = validate_and_cast(Flexible, {"lr": "2", "extra": {"deep": [1]}})
    assert flex["lr"] == 2.0 and flex["extra"] == {"deep": [1]}            # flexible configs keep what they do not know


def test_build_accepts_names_mappings_dataclasses_and_checks_types():
    class Base:
        def __init__(self, cfg, **kw):
            self.cfg, self.kw = cfg, kw

    _, register, build_local = make_registry("t_validation_reg", Base)

    @register("strict", Strict)
    class A(Base):
        pass

    @register("plain")                                                     # no config class: the mapping is passed through
    class B(Base):
        pass

    assert build_local("strict").cfg.lr == 1e-3
    assert build_local({"_name": "strict", "lr": 2}).cfg.lr == 2.0
    assert build_local({"_name": "strict", "lr": 3.0, "inner": Inner(n=5)}).cfg.inner.n == 5     # dataclass instance as a value
    assert build_local({"_name": "plain", "free": 1}, extra=2).kw == {"extra": 2}
    assert build_local(None) is None
    assert isinstance(build_local("strict", cast_to=A), A)
    with pytest.raises(AssertionError):
        build_local("strict", cast_to=B)
    with pytest.raises(KeyError) as err:
        build_local({"_name": "missing"})
    assert "strict" in str(err.value)                                      # the error lists what is registered
    assert isinstance(build("t_validation_reg", "plain"), B)               # module-level build by registry name
    with pytest.raises(KeyError):
        build("no_such_registry", "x")
    with pytest.raises(Exception):
        @register("strict", Strict)
        class Again(Base):
            pass

    @register("not_base")
    class C:                                                               # not a subclass of the registry's base class
        def __init__(self, cfg, **kw):
            pass

    with pytest.raises(AssertionError):
        build_local("not_base")


def test_arch_presets_store_config_instances_that_overrides_refine():
    _, register, build_local = make_registry("t_arch_reg")

    @register("net", Strict)
    class Net:
        def __init__(self, cfg):
            self.cfg = cfg

    @Net.register_arch("small")
    def small():
        return Strict(lr=0.25, tags=["s"])

    @Net.register_arch("large")
    def large():
        return Strict(lr=0.01, inner=Inner(n=9))

    assert build_local("net-small").cfg.tags == ["s"] and build_local("net-large").cfg.inner.n == 9
    refined = build_local({"_name": "net-large", "inner": {"name": "deep"}, "flag": True})
    assert refined.cfg.lr == 0.01 and refined.cfg.inner.n == 9 and refined.cfg.inner.name == "deep" and refined.cfg.flag is True
    assert build_local("net").cfg.lr == 1e-3                               # the plain name keeps the class defaults
