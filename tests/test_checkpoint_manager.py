"""Checkpoint manager: path resolution, save cadence, on-disk layout, latest links, load strategies and
model-only loading (optimus_dl/modules/checkpoint/checkpoint_manager.py:106-814, load_strategy.py:15-85)."""

import os

import pytest
import torch

from optimus_dl_b200.checkpoint.checkpoint_manager import CheckpointManager
from optimus_dl_b200.checkpoint.load_strategy import LoadStrategy
from optimus_dl_b200.lr_scheduler import build_lr_scheduler
from optimus_dl_b200.metrics import base as mb
from optimus_dl_b200.metrics import common as mc
from optimus_dl_b200.models import build_model

MODEL = dict(_name="llama2", n_layer=1, n_head=2, n_kv_head=1, n_embd=32, vocab_size=61, sequence_length=16, multiple_of=8)


class _Loader:
    def __init__(self, pos=0):
        self.pos = pos

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, s):
        self.pos = s["pos"]


def _setup(seed=0, lr=0.1):
    torch.manual_seed(seed)
    model = build_model(MODEL)
    opt = torch.optim.AdamW(model.parameters(), lr=lr)
    sched = build_lr_scheduler({"_name": "wsd", "warmup_steps": 2}, optimizer=opt, iterations=20)
    return model, opt, sched


def _train(model, opt, sched, steps):
    for _ in range(steps):
        loss = model(torch.randint(0, 61, (2, 8)))["logits"].float().logsumexp(-1).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        sched.step()


def _save(mgr, it, model, opt, sched, **kw):
    mgr.save_checkpoint(iteration=it, model=model, optimizer=opt, lr_scheduler=sched, full_config={"model": MODEL}, **kw)


def test_layout_links_and_path_resolution(tmp_path):
    out = tmp_path / "run"
    mgr = CheckpointManager(output_path=str(out))
    assert not mgr.is_restart() and mgr.get_checkpoint(str(out)) is None
    model, opt, sched = _setup()
    _train(model, opt, sched, 2)
    _save(mgr, 5, model, opt, sched, data_loaders={"train": _Loader(7)})
    names = set(os.listdir(out))
    assert {"checkpoint_000000005", "metadata_000000005.pt", "per_rank_metadata_0_000000005.pt", "checkpoint_latest",
            "metadata_latest.pt", "per_rank_metadata_0_latest.pt"} <= names
    assert not [n for n in names if n.endswith(".tmp")]
    assert os.path.islink(out / "metadata_latest.pt") and os.readlink(out / "metadata_latest.pt") == "metadata_000000005.pt"
    assert os.path.exists(out / "checkpoint_000000005" / ".metadata")
    assert mgr.is_restart()
    meta = torch.load(out / "metadata_000000005.pt", weights_only=False)
    assert meta["iteration"] == 5 and meta["world_size"] == 1 and meta["config"]["model"]["n_embd"] == 32
    assert meta["lr_scheduler"]["step_count"] == 2
    # every accepted spelling of "this checkpoint" resolves to the same pair
    want = (str(out / "metadata_000000005.pt"), str(out / "checkpoint_000000005"))
    assert tuple(mgr.get_checkpoint(out / "checkpoint_000000005")) == want
    assert tuple(mgr.get_checkpoint(out / "metadata_000000005.pt")) == want
    latest = mgr.get_checkpoint(out)
    assert latest.metadata.endswith("metadata_latest.pt") and latest.checkpoint.endswith("checkpoint_latest")
    assert tuple(mgr.get_checkpoint(out / "metadata_latest.pt")) == (latest.metadata, latest.checkpoint)
    assert mgr.get_checkpoint(tmp_path / "missing") is None
    with pytest.raises(FileNotFoundError):
        mgr.load_checkpoint(str(tmp_path / "missing"))


def test_save_cadence_persistent_versus_rolling(tmp_path):
    out = tmp_path / "run"
    mgr = CheckpointManager(output_path=str(out))
    model, opt, sched = _setup()
    saved = [it for it in range(1, 13) if mgr.save_checkpoint_if_needed(
        it, save_freq=6, last_save_freq=4, model=model, optimizer=opt, lr_scheduler=sched, full_config={})]
    assert saved == [4, 6, 8, 12]
    names = set(os.listdir(out))
    assert {"checkpoint_000000006", "checkpoint_000000012"} <= names
    assert "checkpoint_000000004" not in names and "checkpoint_000000008" not in names     # rolling saves reuse "latest"
    assert torch.load(out / "metadata_latest.pt", weights_only=False)["iteration"] == 12
    assert not mgr.save_checkpoint_if_needed(13, save_freq=6, last_save_freq=4)
    assert mgr.save_checkpoint_if_needed(13, save_freq=6, last_save_freq=4, force_save=True, model=model, optimizer=opt,
                                         lr_scheduler=sched, full_config={})
    assert "checkpoint_000000013" in os.listdir(out)


def test_full_round_trip_restores_model_optimizer_schedule_loaders_and_meters(tmp_path):
    mgr = CheckpointManager(output_path=str(tmp_path))
    model, opt, sched = _setup()
    _train(model, opt, sched, 3)
    with mb.meters_group("train", log_freq=10):
        mc.log_summed("total_tokens", 123.0, reset=False)
    _save(mgr, 3, model, opt, sched, data_loaders={"train": _Loader(11)})
    want = {k: v.clone() for k, v in model.state_dict().items()}
    mb.clear_all()
    m2, o2, s2 = _setup(seed=1, lr=0.5)
    loader = _Loader()
    start, meta = mgr.load_checkpoint_if_exists(model=m2, optimizer=o2, lr_scheduler=s2, data_loaders={"train": loader})
    assert start == 4 and meta["iteration"] == 3
    assert all(torch.equal(want[k], v) for k, v in m2.state_dict().items())
    assert s2.last_epoch == 3 and o2.param_groups[0]["lr"] == opt.param_groups[0]["lr"]
    assert loader.pos == 11 and mb.compute_meters("train")["total_tokens"] == 123.0
    st1, st2 = opt.state_dict()["state"], o2.state_dict()["state"]
    assert st1.keys() == st2.keys() and all(torch.equal(st1[k]["exp_avg"], st2[k]["exp_avg"]) for k in st1)
    # both copies now take the same next step
    torch.manual_seed(5)
    _train(model, opt, sched, 1)
    torch.manual_seed(5)
    _train(m2, o2, s2, 1)
    assert all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), m2.state_dict().values()))
    # what the reference's loader asks a checkpoint for: every parameter group carries ``param_names`` beside
    # ``params`` (torch records them for optimizers built from named parameters, which the reference's are)
    from optimus_dl_b200.parallel import state as pstate

    exported = pstate.optimizer_state_dict(model, opt, None)
    assert all(g["param_names"] == g["params"] and g["params"] for g in exported["param_groups"])
    assert set(exported["state"]) == {n for n, _ in model.named_parameters()}


def test_load_strategy_switches_each_part_off(tmp_path):
    mgr = CheckpointManager(output_path=str(tmp_path))
    model, opt, sched = _setup()
    _train(model, opt, sched, 3)
    with mb.meters_group("train"):
        mc.log_summed("total_tokens", 9.0, reset=False)
    _save(mgr, 3, model, opt, sched, data_loaders={"train": _Loader(4)})
    mb.clear_all()
    m2, o2, s2 = _setup(seed=1)
    before = {k: v.clone() for k, v in m2.state_dict().items()}
    loader = _Loader()
    strat = LoadStrategy(load_model=True, load_optimizer=False, load_scheduler=False, load_dataloaders=False,
                         load_metrics=False, load_iteration=False)
    meta = mgr.load_checkpoint(str(tmp_path), model=m2, optimizer=o2, lr_scheduler=s2, data_loaders={"train": loader},
                               strategy=strat)
    assert meta["iteration"] == 0                          # a fine-tune starts counting from zero
    assert any(not torch.equal(before[k], v) for k, v in m2.state_dict().items())          # weights did load
    assert s2.last_epoch == 0 and loader.pos == 0 and not o2.state_dict()["state"] and mb.compute_meters("train") == {}
    m3, o3, s3 = _setup(seed=2)
    keep = m3.transformer.ln_f.weight.detach().clone()
    assert not torch.equal(model.transformer.ln_f.weight, keep)
    mgr.load_checkpoint(str(tmp_path), model=m3, strategy={"load_optimizer": False, "extra_ignore_keys": ["ln_f"]})
    assert torch.equal(m3.transformer.ln_f.weight, keep)   # ignored keys keep their fresh initialisation
    assert torch.equal(m3.transformer.h[0].attn.wq.weight, model.transformer.h[0].attn.wq.weight)


def test_metadata_only_save_keeps_the_weights_of_the_full_save(tmp_path):
    mgr = CheckpointManager(output_path=str(tmp_path))
    model, opt, sched = _setup()
    _save(mgr, 2, model, opt, sched)
    stamp = os.path.getmtime(tmp_path / "checkpoint_000000002" / ".metadata")
    mgr.save_checkpoint(iteration=2, lr_scheduler=sched, full_config={"model": MODEL}, metadata_only=True,
                        extra_metadata={"eval_finished": True})
    meta = torch.load(tmp_path / "metadata_000000002.pt", weights_only=False)
    assert meta["eval_finished"] is True
    assert os.path.getmtime(tmp_path / "checkpoint_000000002" / ".metadata") == stamp
    assert os.path.exists(tmp_path / "per_rank_metadata_0_000000002.pt")


def test_model_can_be_rebuilt_from_the_checkpoint_alone(tmp_path):
    mgr = CheckpointManager(output_path=str(tmp_path))
    model, opt, sched = _setup()
    _train(model, opt, sched, 1)
    _save(mgr, 1, model, opt, sched)
    rebuilt, meta = CheckpointManager().build_model_from_checkpoint(str(tmp_path))
    assert meta["iteration"] == 1 and type(rebuilt) is type(model)
    x = torch.randint(0, 61, (1, 8))
    assert torch.equal(rebuilt.eval()(x)["logits"], model.eval()(x)["logits"])
    plain = tmp_path / "weights.pt"
    torch.save(model.state_dict(), plain)
    other = build_model(MODEL)
    CheckpointManager().load_model_state_dict(other, str(plain))
    assert torch.equal(other.lm_head.weight, model.lm_head.weight)


def test_checkpoint_path_helpers_and_eval_state_cleanup(tmp_path):
    from optimus_dl_b200.checkpoint.eval_checkpoint_manager import EvaluationCheckpointManager

    mgr = CheckpointManager(output_path=str(tmp_path))
    model, opt, sched = _setup()
    _save(mgr, 4, model, opt, sched)
    cp = mgr.get_checkpoint(tmp_path / "metadata_000000004.pt")
    assert cp.is_dcp_checkpoint() and cp.per_rank_metadata(0) == str(tmp_path / "per_rank_metadata_0_000000004.pt")
    assert os.path.exists(cp.per_rank_metadata(0)) and cp.per_rank_metadata(3).endswith("per_rank_metadata_3_000000004.pt")
    ev = EvaluationCheckpointManager(str(tmp_path), rank=0)
    from optimus_dl_b200.metrics.base import meters_group
    from optimus_dl_b200.metrics.common import log_summed
    with meters_group("eval/tiny", log_freq=1, force_recreate=True):
        log_summed("num_batches", lambda: 2)
    for it in (10, 20, 30):
        ev.save_iteration_state(it, "tiny", {"pos": it}, "eval/tiny", eval_iterations_processed=2)
    assert ev.get_eval_checkpoints_dir(20).name == "eval_checkpoints_iter_20" and ev.get_eval_checkpoints_dir(20).is_dir()
    assert ev.read_iteration_state(20, "tiny")["dataloader_state"] == {"pos": 20}
    assert ev.load_iteration_state(20, "tiny", "eval/tiny") == 2
    ev.cleanup(iteration=10)
    assert not ev.get_eval_checkpoints_dir(10).exists() and ev.get_eval_checkpoints_dir(20).exists()
    ev.cleanup(exclude_iteration=30)
    assert not ev.get_eval_checkpoints_dir(20).exists() and ev.get_eval_checkpoints_dir(30).exists()
    ev.cleanup()
    assert not ev.get_eval_checkpoints_dir(30).exists()


def test_reference_call_forms_of_the_manager(tmp_path):
    """Keyword names of optimus_dl/modules/checkpoint/checkpoint_manager.py:78-835: ``checkpoint_path``,
    ``is_save_persistent`` / ``is_save_last``, ``load_strategy``, and ``(iteration, collective, path)`` positionally."""
    from unittest.mock import patch

    from optimus_dl_b200.parallel.collective import FakeCollective

    coll = FakeCollective(rank=0, world_size=1)
    mgr = CheckpointManager()
    with patch.object(mgr, "save_checkpoint") as save:
        assert mgr.save_checkpoint_if_needed(10, coll, "tmp", save_freq=10, last_save_freq=None)
        kw = save.call_args.kwargs
        assert kw["is_save_persistent"] is True and kw["is_save_last"] is True and kw["checkpoint_path"] == "tmp"
        save.reset_mock()
        assert not mgr.save_checkpoint_if_needed(5, coll, "tmp", save_freq=10, last_save_freq=None)
        save.assert_not_called()
        assert mgr.save_checkpoint_if_needed(5, coll, "tmp", save_freq=10, last_save_freq=5)
        assert save.call_args.kwargs["is_save_persistent"] is False and save.call_args.kwargs["is_save_last"] is True
    model = torch.nn.Linear(4, 4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    root = tmp_path / "checkpoints"
    mgr.save_checkpoint(checkpoint_path=root, model=model, optimizer=opt, collective=coll, full_config={},
                        is_save_persistent=True, is_save_last=True, iteration=10)
    assert (root / "checkpoint_latest").is_symlink() and (root / "metadata_latest.pt").is_symlink()
    assert (root / "per_rank_metadata_0_latest.pt").is_symlink() and os.readlink(root / "checkpoint_latest") == "checkpoint_000000010"
    other = tmp_path / "last_only"
    mgr.save_checkpoint(checkpoint_path=other, model=model, optimizer=opt, collective=coll, full_config={},
                        is_save_persistent=False, is_save_last=True, iteration=15)
    assert (other / "checkpoint_latest").is_dir() and not (other / "checkpoint_latest").is_symlink()
    assert not list(other.glob("checkpoint_0*")) and (other / "metadata_latest.pt").exists()
    fresh = torch.nn.Linear(4, 4)
    loader = CheckpointManager()
    assert loader.is_restart(other) and not loader.is_restart(tmp_path / "nothing")
    start, meta = loader.load_checkpoint_if_exists(checkpoint_path=other, model=fresh, optimizer=None, collective=coll,
                                                    load_strategy=None)
    assert start == 16 and meta["iteration"] == 15 and torch.equal(fresh.weight, model.weight)
    assert loader.load_checkpoint_if_exists(checkpoint_path=tmp_path / "nothing", model=fresh) == (1, None)
