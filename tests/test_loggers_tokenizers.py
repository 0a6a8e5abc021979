"""JSONL metrics logger, the logger manager, and the tokenizers that need no download
(optimus_dl/modules/loggers/jsonl.py:30-373, optimus_dl/recipe/train/mixins/managers/logger_manager.py:23-206,
optimus_dl/modules/tokenizer/implementations/{char,inline_tokens}.py)."""

import json
import os

import pytest
import torch
import yaml

from optimus_dl_b200.loggers import build_metrics_logger
from optimus_dl_b200.loggers.base import RunStatus, flatten_metrics
from optimus_dl_b200.metrics import base as mb
from optimus_dl_b200.recipe.train.mixins.managers.logger_manager import LoggerManager
from optimus_dl_b200.tokenizer import build_tokenizer


def _lines(path):
    with open(path) as f:
        return [json.loads(x) for x in f if x.strip()]


def test_jsonl_writes_one_file_per_group_and_dumps_the_config(tmp_path):
    lg = build_metrics_logger({"_name": "jsonl", "output_dir": str(tmp_path / "logs"), "flush_every": 1})
    lg.setup("exp", {"model": {"n_layer": 2}, "lr": 1e-3, "dtype": torch.bfloat16}, logs_parent_path=None, start_iteration=1)
    lg.log_metrics({"loss": torch.tensor(2.5), "nested": {"a": 1}, "items": (1, 2)}, step=1)
    lg.log_metrics({"loss": 2.0}, step=2)
    lg.log_metrics({"accuracy": 0.5}, step=2, group="eval/tiny")
    lg.finished(RunStatus.FINISHED)
    lg.close()
    d = tmp_path / "logs"
    train = _lines(d / "metrics.jsonl")
    assert [r["step"] for r in train] == [1, 2] and train[0]["loss"] == 2.5 and train[0]["group"] == "train"
    assert train[0]["nested_a"] == 1 and train[0]["items"] == [1, 2]            # dictionaries flatten one level
    assert "T" in train[0]["timestamp"] and list(train[0])[:3] == ["step", "group", "timestamp"]
    ev = _lines(d / "metrics_eval_tiny.jsonl")
    assert len(ev) == 1 and ev[0]["accuracy"] == 0.5 and ev[0]["group"] == "eval/tiny"
    final = _lines(d / "metrics_final.jsonl")[0]
    assert final["status"] == "success" and final["group"] == "final" and final["step"] is None
    assert RunStatus.FINISHED is RunStatus.SUCCESS and RunStatus.FAILED is RunStatus.FAILURE
    assert RunStatus("interrupted") is RunStatus.INTERRUPTED
    cfg_json = json.load(open(d / "exp_config.json"))
    assert cfg_json["model"]["n_layer"] == 2 and cfg_json["dtype"] == "torch.bfloat16"
    assert yaml.safe_load(open(d / "exp_config.yaml"))["lr"] == 1e-3


def test_jsonl_options_single_file_no_timestamp_sorted_truncate(tmp_path):
    cfg = {"_name": "jsonl", "output_dir": str(tmp_path), "filename": "run.log", "include_group_in_filename": False,
           "include_timestamp": False, "sort_keys": True, "dump_config": False, "append_mode": False}
    (tmp_path / "run.log").write_text("stale\n")
    lg = build_metrics_logger(cfg)
    lg.setup("exp", {})
    lg.log_metrics({"z": 1, "a": 2}, step=1)
    lg.log_metrics({"b": 3}, step=1, group="eval")
    lg.close()
    text = (tmp_path / "run.log").read_text().splitlines()
    assert text == ['{"a": 2, "group": "train", "step": 1, "z": 1}', '{"b": 3, "group": "eval", "step": 1}']
    assert sorted(os.listdir(tmp_path)) == ["run.log"]


def test_jsonl_rotation_keeps_the_newest_lines_in_the_plain_file(tmp_path):
    cfg = {"_name": "jsonl", "output_dir": str(tmp_path), "max_file_size_mb": 0.001, "max_rotated_files": 2,
           "dump_config": False, "include_timestamp": False}
    lg = build_metrics_logger(cfg)
    lg.setup("exp", {})
    for step in range(60):
        lg.log_metrics({"loss": float(step), "pad": "x" * 100}, step=step)
    lg.close()
    parts = sorted(os.listdir(tmp_path))
    assert parts == ["metrics.1.jsonl", "metrics.2.jsonl", "metrics.jsonl"]       # older parts were dropped
    newest = [r["step"] for r in _lines(tmp_path / "metrics.jsonl")]
    mid = [r["step"] for r in _lines(tmp_path / "metrics.1.jsonl")]
    old = [r["step"] for r in _lines(tmp_path / "metrics.2.jsonl")]
    assert newest[-1] == 59 and old + mid + newest == list(range(old[0], 60))      # contiguous, newest last
    again = build_metrics_logger(cfg)                                               # a restart appends to the plain file
    again.setup("exp", {})
    again.log_metrics({"loss": -1.0}, step=60)
    again.close()
    assert _lines(tmp_path / "metrics.jsonl")[-1]["step"] == 60
    unlimited = build_metrics_logger({**cfg, "output_dir": str(tmp_path / "u"), "max_rotated_files": -1})
    unlimited.setup("exp", {})
    for step in range(60):
        unlimited.log_metrics({"loss": float(step), "pad": "x" * 100}, step=step)
    unlimited.close()
    all_steps = []
    files = sorted(os.listdir(tmp_path / "u"), key=lambda n: -int(n.split(".")[1]) if n.count(".") == 2 else 1)
    for n in files:
        all_steps += [r["step"] for r in _lines(tmp_path / "u" / n)]
    assert all_steps == list(range(60)) and len(files) > 3                          # nothing is ever deleted


def test_disabled_logger_writes_nothing(tmp_path):
    lg = build_metrics_logger({"_name": "jsonl", "output_dir": str(tmp_path / "off"), "enabled": False})
    lg.setup("exp", {"a": 1})
    lg.log_metrics({"loss": 1.0}, step=1)
    lg.finished()
    lg.close()
    assert not os.path.exists(tmp_path / "off")


def test_flatten_metrics_joins_nested_keys():
    assert flatten_metrics({"a": 1, "b": {"c": 2, "d": {"e": 3}}}) == {"a": 1, "b/c": 2, "b/d/e": 3}


class _Boom:
    cfg = {"_name": "boom"}

    def setup(self, *a):
        raise RuntimeError("setup")

    def log_metrics(self, *a):
        raise RuntimeError("log")

    def finished(self, *a):
        raise RuntimeError("finished")

    def close(self):
        raise RuntimeError("close")

    def state_dict(self):
        return {"k": 1}

    def load_state_dict(self, s):
        self.loaded = s


def test_logger_manager_isolates_failures_keys_state_by_id_and_times_itself(tmp_path):
    mgr = LoggerManager(loggers_config=[
        {"_name": "jsonl", "output_dir": str(tmp_path / "a"), "dump_config": False},
        {"_name": "jsonl", "id": "second", "output_dir": str(tmp_path / "b"), "dump_config": False},
        {"_name": "jsonl", "output_dir": str(tmp_path / "c"), "enabled": False},
    ])
    mgr.build_loggers()
    assert len(mgr.loggers) == 2                         # disabled entries are not built
    mgr.loggers.append(_Boom())
    mgr.setup_loggers("exp", {})
    with mb.meters_group("train", log_freq=1):
        mgr.log_metrics_to_loggers({"loss": 1.0}, step=3)
        assert mb.compute_meters("train")["ms_spent_logging"] >= 0.0
    mgr.finished()
    mgr.close_loggers()                                  # the failing logger never stops the others
    assert _lines(tmp_path / "a" / "metrics.jsonl")[0]["step"] == 3 and _lines(tmp_path / "b" / "metrics.jsonl")[0]["loss"] == 1.0
    sd = mgr.state_dict()
    assert set(sd) == {"jsonl", "second", "boom"} and sd["boom"] == {"k": 1} and sd["jsonl"] == {}
    seen = {}
    from optimus_dl_b200.loggers import register_metrics_logger
    from optimus_dl_b200.loggers.base import BaseMetricsLogger
    from optimus_dl_b200.loggers.config import MetricsLoggerConfig

    class _Remember(BaseMetricsLogger):
        def __init__(self, cfg, state_dict=None, **kw):
            super().__init__(cfg)
            seen["state"] = state_dict

    try:
        register_metrics_logger("t_remember", MetricsLoggerConfig)(_Remember)
    except (AssertionError, ValueError, KeyError):
        pass
    fresh = LoggerManager(loggers_config=[{"_name": "t_remember", "id": "second"}])
    fresh.load_state_dict({"second": {"run_id": "abc"}})
    fresh.build_loggers()                                # state given before building reaches the constructor
    assert seen["state"] == {"run_id": "abc"}


def test_char_tokenizer_round_trips_utf8_and_reserves_bos_eos():
    tok = build_tokenizer({"_name": "char_tokenize"})
    ids = tok.encode("añ€")
    assert ids[0] == tok.bos_token_id == 256 and ids[-1] == tok.eos_token_id == 257 and tok.vocab_size >= 258
    assert ids[1:-1] == list("añ€".encode())
    assert tok.decode(ids) == "añ€"                      # special ids vanish on decode
    bare = build_tokenizer({"_name": "char_tokenize", "add_bos": False, "add_eos": False})
    assert bare.encode("hi") == [104, 105]
    chat = bare.apply_chat_template([{"role": "user", "content": "2+2?"}], tokenize=False)
    assert chat == "user: 2+2?\nassistant:"
    assert bare.apply_chat_template([{"role": "user", "content": "x"}], add_generation_prompt=False) == bare.encode("user: x\n")
    with pytest.raises(NotImplementedError):
        bare.save_pretrained("/nonexistent")


def test_inline_tokens_longest_match_and_unknown_policies():
    vocab = ["a", "ab", "abc", " ", "+"]
    tok = build_tokenizer({"_name": "inline_tokens_tokenizer", "tokens": vocab})
    assert tok.vocab_size == 7 and tok.bos_token_id == 5 and tok.eos_token_id == 6
    assert tok.encode("abcab a+") == [5, 2, 1, 3, 0, 4, 6]          # longest token wins at each position
    assert tok.decode(tok.encode("abcab a+")) == "abcab a+"
    with pytest.raises(ValueError):
        tok.encode("abz")
    ign = build_tokenizer({"_name": "inline_tokens_tokenizer", "tokens": vocab, "unk_strategy": "ignore", "add_bos": False,
                           "add_eos": False})
    assert ign.encode("azzb+") == [0, 4] and ign.vocab_size == 7
    unk = build_tokenizer({"_name": "inline_tokens_tokenizer", "tokens": vocab, "unk_strategy": "unk", "add_bos": False,
                           "add_eos": False})
    assert unk.vocab_size == 8 and unk.encode("a?b+") == [0, 7, 7, 4] or unk.encode("a?b+") == [0, 7, 4]
    assert "<UNK>" in unk.decode(unk.encode("a?+")) and unk._unk_token_id == 7 and tok._unk_token_id is None
    with pytest.raises(ValueError, match="Invalid token ID: 99"):
        tok.decode([5, 99, 6])
    with pytest.raises(ValueError, match="Unknown token/characters encountered"):
        tok.encode("abXYZ")
    wide = build_tokenizer({"_name": "inline_tokens_tokenizer", "tokens": ["A", "B", "C", "AB", "BC", "word", "!"], "unk_strategy": "unk"})
    assert wide.encode("$A$") == [7, 9, 0, 9, 8] and wide.encode("ABXYZC") == [7, 3, 9, 2, 8]   # a run of unknown text is one UNK
    assert wide.decode([7, 3, 9, 2, 8]) == "AB<UNK>C"
    dotted = build_tokenizer({"_name": "inline_tokens_tokenizer", "tokens": [".", "*", "a"], "add_bos": False, "add_eos": False})
    assert dotted.encode("a.*") == [2, 0, 1]                          # vocabulary entries are literals, not patterns
