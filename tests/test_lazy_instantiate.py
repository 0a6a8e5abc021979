"""Lazy, reactive ``_target_`` instantiation and the config tree it lives in
(optimus_dl/core/omegaconf_utils.py:146-482), one behaviour per test."""

import pytest

from optimus_dl_b200.core import conf
from optimus_dl_b200.core.config_utils import non_resolving_instantiate as nri

from tests import _lazy_targets as LT

COUNT = LT.COUNT
T = "tests._lazy_targets"


@pytest.fixture(autouse=True)
def _reset():
    COUNT["n"] = 0
    yield


def test_target_runs_on_first_access_and_not_before():
    c = nri({"obj": {"_target_": f"{T}.make", "x": 1}, "plain": 5})
    assert COUNT["n"] == 0 and c.plain == 5 and COUNT["n"] == 0
    assert c.obj["x"] == 1 and COUNT["n"] == 1
    assert c.obj["_call"] == 1 and COUNT["n"] == 1                  # the built object is cached while nothing changes


def test_object_is_rebuilt_when_a_value_it_interpolates_changes():
    c = nri({"base": {"lr": 0.1}, "opt": {"_target_": f"{T}.make", "lr": "${base.lr}", "fixed": 3}})
    assert c.opt["lr"] == 0.1 and c.opt["_call"] == 1
    c.base.lr = 0.2
    assert c.opt["lr"] == 0.2 and c.opt["_call"] == 2 and c.opt["fixed"] == 3
    c.base.other = 1                                                  # unrelated edits do not rebuild
    assert c.opt["_call"] == 2


def test_relative_interpolations_inside_a_target_resolve_from_its_position():
    c = nri({"group": {"width": 8, "layer": {"_target_": f"{T}.make", "w": "${..width}", "twice": "${eval:'${..width} * 2'}"}},
             "width": 99})
    assert c.group.layer["w"] == 8 and c.group.layer["twice"] == 16
    c.group.width = 5
    assert c.group.layer["w"] == 5 and c.group.layer["twice"] == 10


def test_targets_nest_and_inner_objects_are_built_first():
    c = nri({"outer": {"_target_": f"{T}.make", "inner": {"_target_": f"{T}.make", "v": "${scale}"}, "tag": "o"}, "scale": 2})
    o = c.outer
    assert o["tag"] == "o" and o["inner"]["v"] == 2 and o["inner"]["_call"] < o["_call"]
    c.scale = 3
    assert c.outer["inner"]["v"] == 3


def test_positional_arguments_and_partial():
    c = nri({"s": {"_target_": f"{T}.add", "_args_": [2, 5]}, "p": {"_target_": f"{T}.add", "_partial_": True, "b": 10}})
    assert c.s == 7
    assert c.p(1) == 11 and c.p(a=5) == 15


def test_references_to_a_lazy_object_share_the_instance():
    c = nri({"model": {"_target_": f"{T}.make", "d": 4}, "a": "${model}", "nested": {"b": "${model}"}})
    assert c.a is c.nested.b and c.a["_call"] == 1 and COUNT["n"] == 1


def test_list_items_may_be_targets_and_may_reference_siblings():
    c = nri({"items": [{"_target_": f"{T}.add", "_args_": [1, 1]}, "${.0}", {"_target_": f"{T}.add", "_args_": ["${base}", 1]}],
             "base": 10})
    assert c["items"][0] == 2 and c["items"][1] == 2 and c["items"][2] == 11
    c.base = 20
    assert c["items"][2] == 21


def test_cycles_between_lazy_objects_are_reported():
    c = nri({"a": {"_target_": f"{T}.make", "x": "${b}"}, "b": {"_target_": f"{T}.make", "y": "${a}"}})
    with pytest.raises(conf.InterpolationError):
        c.a
    self_ref = nri({"a": {"_target_": f"{T}.make", "me": "${a}"}})
    with pytest.raises(conf.InterpolationError):
        self_ref.a


def test_eager_mode_builds_everything_at_once():
    c = nri({"a": {"_target_": f"{T}.make", "v": 1}, "b": {"_target_": f"{T}.make", "v": "${a}"}}, lazy=False)
    assert COUNT["n"] >= 2 and c.b["v"]["v"] == 1


def test_unknown_targets_and_failing_targets_raise_on_access_only():
    c = nri({"bad": {"_target_": "no.such.module.fn"}, "boom": {"_target_": "builtins.int", "_args_": ["x"]}, "ok": 1})
    assert c.ok == 1
    with pytest.raises(Exception):
        c.bad
    with pytest.raises(Exception):
        c.boom


def test_to_container_keeps_definitions_unresolved_and_resolves_on_request():
    raw = {"p": 2, "o": {"_target_": f"{T}.add", "_args_": ["${p}", 1]}, "s": "${p}"}
    c = nri(conf.create(raw))
    assert conf.to_container(c, resolve=False)["s"] == "${p}"
    assert conf.to_container(c, resolve=True)["s"] == 2
    assert c.o == 3


def test_helpers_are_usable_as_targets():
    c = nri({"sizes": {"_target_": "optimus_dl_b200.core.instantiate.repeat", "item": 64, "times": 3},
             "all": {"_target_": "optimus_dl_b200.core.instantiate.concat_lists", "_args_": ["${sizes}", [1]]},
             "pick": {"_target_": "optimus_dl_b200.core.instantiate.cond", "condition": "${flag}", "true_val": "yes", "false_val": "no"},
             "flag": False})
    assert c.sizes == [64, 64, 64] and c["all"] == [64, 64, 64, 1] and c.pick == "no"
    c.flag = True
    assert c.pick == "yes"


def test_helper_signatures_and_semantics():
    """Call forms of optimus_dl/core/instantiate.py:19-175."""
    from optimus_dl_b200.core.instantiate import compose, concat_lists, cond, get_item, merge_dicts, repeat

    merged = merge_dicts({"a": 1, "b": {"c": 2}}, {"b": {"d": 3}, "e": 4}, conf.create({"a": 10, "f": 5}))
    assert merged == {"a": 10, "b": {"c": 2, "d": 3}, "e": 4, "f": 5}                 # deep merge, later arguments win
    assert cond(True, "foo", "bar") == "foo" and cond(False, "foo", "bar") == "bar" and cond(True, {"a": 1}, [1, 2]) == {"a": 1}
    assert cond(False, if_true=1, if_false=2) == 2
    base = {"_target_": "module", "layer": 1}
    copies = repeat(3, base)
    copies[0]["layer"] = 2
    assert len(copies) == 3 and copies[1] == base and copies[2]["layer"] == 1          # independent deep copies
    assert repeat(value=7, times=2) == [7, 7] and repeat([1], 2) == [[1], [1]]
    assert concat_lists([1, 2, 3], conf.create([4, 5]), [6]) == [1, 2, 3, 4, 5, 6]
    with pytest.raises(ValueError):
        concat_lists([1], {"a": 1})
    table = {"adam": "AdamW", "sgd": "SGD"}
    assert get_item("adam", table) == "AdamW" and get_item("sgd", conf.create(table)) == "SGD"
    assert get_item("rmsprop", table, default="Missing") == "Missing" and get_item(table, "adam") == "AdamW"
    with pytest.raises(KeyError):
        get_item("rmsprop", table)
    pipeline = compose(lambda x: x + 1, lambda x: x * 2, str)
    assert pipeline(3) == "8" and compose()(42) == 42
    assert compose(lambda a, b=2: {"a": a, "b": b}, lambda d: d["b"])(5, b=10) == 10   # the first function gets every argument
    with pytest.raises(ValueError):
        compose()(1, 2)


def test_braces_between_quotes_do_not_close_an_interpolation():
    """optimus_dl/core/omegaconf_utils.py (_extract_interpolations): quoted text inside ``${...}`` is text."""
    c = nri(conf.create({"a": "}", "obj": {"_target_": "builtins.dict", "val": "${eval:'\"}\"'}"}}))
    assert c.obj["val"] == "}"
    c = nri(conf.create({"x": "hello", "obj": {"_target_": "builtins.dict", "val": '${eval:\'"} " + "${x}" + " {"\'}'}}))
    assert c.obj["val"] == "} hello {"
    c.x = "bye"
    assert c.obj["val"] == "} bye {"                                                    # the dependency inside the quotes is tracked
    plain = conf.create({"h": "it's", "v": "${oc.env:OPTIMUS_NO_SUCH_VARIABLE,it's}", "w": "a ${h} b ${eval:'1+1'}"})
    assert plain.v == "it's" and plain.w == "a it's b 2"                                # a lone apostrophe is still text


def test_relative_reference_to_a_sibling_key_of_the_target_and_root_targets():
    c = nri(conf.create({"a": {"b": {"c": {"_target_": "builtins.dict", "val": "${.d}", "d": 42}}}}))
    assert c.a.b.c["val"] == 42
    root = nri(conf.create({"_target_": "builtins.dict", "key": "value"}))
    assert isinstance(root, dict) and not conf.is_config(root) and root == {"key": "value"}
