"""End-to-end behaviour on CPU: script runs, bit-exact resume, failed saves, evaluation resume,
two-rank Gloo collectives."""

import json
import os
import subprocess
import sys
from pathlib import Path
from unittest import mock

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
TINY = ["~lr_scheduler", "model._name=llama2", "+model.n_layer=1", "+model.n_head=2", "+model.n_embd=32", "args.vocab_size=128",
        "args.batch_size=2", "args.seq_len=16", "common.use_gpu=false", "common.eval_freq=0"]


def _train(out: Path, *overrides: str) -> None:
    env = dict(os.environ, SCRATCH_HOME=str(out), OPTIMUS_EXIT_TIMEOUT="0")
    cmd = [sys.executable, str(ROOT / "scripts" / "train.py"), "--config-name=train_synthetic", "common.exp_name=run", *TINY, *overrides]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


def _load_full(run_dir: Path):
    from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

    f = run_dir / "full.pt"
    dcp_to_torch_save(str(run_dir / "checkpoint_latest"), str(f))
    return torch.load(f, weights_only=False)


def _flatten(d, prefix=""):
    out = {}
    for k, v in d.items():
        if isinstance(v, dict):
            out.update(_flatten(v, f"{prefix}{k}."))
        else:
            out[f"{prefix}{k}"] = v
    return out


def test_resume_is_bit_identical_to_uninterrupted_run(tmp_path):
    a, b = tmp_path / "a", tmp_path / "b"
    _train(a, "args.iterations=10", "common.save_freq=10")
    _train(b, "args.iterations=10", "common.save_freq=5", "optimization.iterations=5")
    _train(b, "args.iterations=10", "common.save_freq=5")
    ra, rb = a / "outputs/synthetic/run", b / "outputs/synthetic/run"
    fa, fb = _flatten(_load_full(ra)), _flatten(_load_full(rb))
    assert fa.keys() == fb.keys() and any(k.startswith("optimizer.") for k in fa)
    for k in fa:
        if torch.is_tensor(fa[k]):
            assert torch.equal(fa[k], fb[k]), k
    ma = torch.load(ra / "metadata_latest.pt", weights_only=False)
    assert ma["iteration"] == 10 and ma["config"]["model"]["n_embd"] == 32
    la = [json.loads(l) for l in open(ra / "logs/metrics.jsonl")]
    lb = [json.loads(l) for l in open(rb / "logs/metrics.jsonl")]
    assert [r["loss"] for r in la if r["group"] == "train"] == [r["loss"] for r in lb if r["group"] == "train"]
    assert sorted(p.name for p in rb.iterdir() if p.name.startswith("checkpoint_0")) == ["checkpoint_000000005", "checkpoint_000000010"]
    assert os.path.islink(rb / "checkpoint_latest") and os.readlink(rb / "checkpoint_latest") == "checkpoint_000000010"


def test_failed_save_keeps_previous_latest(tmp_path):
    from optimus_dl_b200.checkpoint import CheckpointManager, checkpoint_manager as cm
    from optimus_dl_b200.models import build_model

    model = build_model(dict(_name="llama2", n_layer=1, n_head=2, n_embd=32, vocab_size=64, sequence_length=16, multiple_of=8))
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    mgr = CheckpointManager(None, output_path=str(tmp_path))
    mgr.save_checkpoint(1, model=model, optimizer=opt, full_config={"model": {"_name": "llama2"}})
    before = torch.load(tmp_path / "metadata_latest.pt", weights_only=False)
    with mock.patch.object(cm, "dcp_save", side_effect=RuntimeError("disk full")):
        with pytest.raises(RuntimeError):
            mgr.save_checkpoint(2, model=model, optimizer=opt, full_config={})
    with mock.patch.object(cm.torch, "save", side_effect=RuntimeError("disk full")):
        with pytest.raises(BaseException):
            mgr.save_checkpoint(3, model=model, optimizer=opt, full_config={})
    after = torch.load(tmp_path / "metadata_latest.pt", weights_only=False)
    assert before["iteration"] == after["iteration"] == 1 and os.readlink(tmp_path / "checkpoint_latest") == "checkpoint_000000001"
    assert mgr.is_restart() and mgr.get_checkpoint(tmp_path).checkpoint.endswith("checkpoint_latest")
    with torch.no_grad():
        for p in model.parameters():
            p.add_(1.0)
    mgr.load_checkpoint(str(tmp_path), model=model, optimizer=opt)
    fresh = build_model(dict(_name="llama2", n_layer=1, n_head=2, n_embd=32, vocab_size=64, sequence_length=16, multiple_of=8))
    mgr.load_model_state_dict(fresh, str(tmp_path / "checkpoint_latest"))
    for (n, p), (_, q) in zip(model.named_parameters(), fresh.named_parameters()):
        assert torch.equal(p, q), n


class CrashMidEval(Exception):
    pass


def test_evaluation_resumes_mid_way_with_same_result(tmp_path):
    """An evaluation that dies after k batches continues from its per-rank checkpoint and ends with the
    metrics of an uninterrupted evaluation."""
    from optimus_dl_b200.checkpoint import EvaluationCheckpointManager
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.data import build_data_pipeline
    from optimus_dl_b200.models import build_model
    from optimus_dl_b200.recipe.train.builders.data_builder import LoaderIterResettable
    from optimus_dl_b200.recipe.train.mixins.managers.evaluation_manager import Evaluator

    torch.manual_seed(0)
    model = build_model(dict(_name="llama2", n_layer=1, n_head=2, n_embd=32, vocab_size=64, sequence_length=16, multiple_of=8))
    crit = build_criterion({"_name": "cross_entropy"})
    cfg = {"source": {"_name": "synthetic_tokens", "vocab_size": 64, "length": 17, "num_documents": 24},
           "transform": {"_name": "flat_batcher", "batch_size": 2, "seq_len": 16}, "eval_iterations": None}

    def pipes():
        p = build_data_pipeline(cfg, eval_pipeline=True, rank=0, world_size=1, seed=0)
        return {"val": p._replace(dataloader=LoaderIterResettable(p.dataloader))}

    ref = Evaluator(eval_freq=1).run_evaluation(model, crit, pipes(), 1)["eval/val"]

    class Crashing:
        def __init__(self, inner, at):
            self.inner, self.n, self.at = inner, 0, at

        def __call__(self, *a, **k):
            self.n += 1
            if self.n == self.at:
                raise CrashMidEval()
            return self.inner(*a, **k)

    ev = Evaluator(eval_freq=1, eval_checkpointing=2, eval_checkpoint_manager=EvaluationCheckpointManager(str(tmp_path), 0))
    with pytest.raises(CrashMidEval):
        ev.run_evaluation(model, Crashing(crit, 6), pipes(), 1)
    assert (tmp_path / "eval_checkpoints_iter_1" / "val_rank_0.pt").exists()
    resumed = ev.run_evaluation(model, crit, pipes(), 1)["eval/val"]
    assert resumed["loss"] == pytest.approx(ref["loss"], abs=1e-4) and resumed["batch_tokens"] == ref["batch_tokens"]


WORKER = r'''
import os, sys, torch
sys.path.insert(0, sys.argv[1])
from optimus_dl_b200.parallel import build_best_collective
from optimus_dl_b200.parallel.collective import DistributedConfig, MeshCollective
from optimus_dl_b200.metrics import meters_group, log_averaged, log_summed, compute_meters
c = build_best_collective(DistributedConfig(tp_size=2, sharding_world_size=1), torch.device("cpu"))
assert isinstance(c, MeshCollective) and c.world_size == 2 and c.tp_world_size == 2 and c.dp_world_size == 1
assert c.tp_rank == c.rank and c.dp_rank == 0 and c.tp_world.world_size == 2
t = torch.tensor([float(c.rank + 1)]); c.all_reduce(t); assert t.item() == 3.0
out = torch.zeros(2); c.all_gather(out, torch.tensor([float(c.rank)])); assert out.tolist() == [0.0, 1.0]
objs = c.all_gather_objects({"r": c.rank}); assert [o["r"] for o in objs] == [0, 1]
box = [{"x": 5} if c.rank == 0 else None]; c.broadcast_objects(box, src=0); assert box[0] == {"x": 5}
with meters_group("g", log_freq=1):
    log_averaged("loss", float(c.rank), weight=1 + c.rank)
    log_summed("tokens", 10.0)
m = compute_meters("g", aggregate=True, collective=c)
assert abs(m["loss"] - (0 * 1 + 1 * 2) / 3) < 1e-9 and m["tokens"] == 20.0
c.close()
print("WORKER_OK", c.rank)
'''


def test_two_rank_gloo_collective_and_meter_aggregation(tmp_path, unique_port):
    script = tmp_path / "w.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(unique_port), str(script), str(ROOT)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0 and res.stdout.count("WORKER_OK") == 2, res.stdout[-2000:] + res.stderr[-3000:]


@pytest.mark.slow
def test_gpt2_small_cpu_oracle_loss_decreases():
    """GPT-2 small, fp32, CPU, batch 4 x 256 uniform tokens, AdamW(3e-4, 0.9/0.95, wd 0.1): the CPU oracle config."""
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.models import build_model
    from optimus_dl_b200.optim import build_optimizer

    torch.manual_seed(0)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    model = build_model(dict(_name="gpt2", n_layer=12, n_head=12, n_embd=768, vocab_size=50257, block_size=1024))
    opt = build_optimizer({"_name": "adamw", "lr": 3e-4, "betas": [0.9, 0.95], "weight_decay": 0.1}, params=model.make_parameter_groups())
    crit = build_criterion({"_name": "cross_entropy"})
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 50257, (4, 257), generator=gen)
    losses = []
    for _ in range(4):
        opt.zero_grad()
        loss, _ = crit(model, {"input_ids": ids})
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert abs(losses[0] - 10.9) < 0.3 and losses[-1] < losses[0]


def test_recipe_exposes_its_builders_and_validates_the_config(tmp_path, monkeypatch):
    """The recipe forwards build / save / load / log calls to its injected parts and refuses a run that cannot train."""
    from optimus_dl_b200.core import compose
    from optimus_dl_b200.core.config_utils import non_resolving_instantiate
    from optimus_dl_b200.core.registry import build

    monkeypatch.setenv("SCRATCH_HOME", str(tmp_path))
    raw = compose.compose([str(ROOT / "configs" / "train")], "train_synthetic", ["common.exp_name=r", *TINY], apply_env=False)
    recipe = build("train_recipe", non_resolving_instantiate(raw))
    recipe.validate_config()
    crit = recipe.build_criterion()
    model = recipe.build_model(recipe.cfg.model, device=torch.device("cpu"))
    opt = recipe.build_optimizer(model.make_parameter_groups())
    assert type(crit).__name__ == "CrossEntropyCriterion" and sum(p.numel() for p in model.parameters()) > 0
    assert len(opt.param_groups) >= 1
    recipe.build_loggers()
    recipe.setup_loggers("r")
    recipe.log_metrics_to_loggers({"loss": 1.0}, 1, "train")
    recipe.close_loggers()
    logs = [p for p in Path(recipe.output_path).rglob("metrics*.jsonl")]
    assert logs and any("final" in p.name for p in logs)
    assert recipe.save_checkpoint_if_needed(3, save_freq=5) is False
    assert recipe.load_checkpoint_if_exists()[0] == 1          # nothing saved yet: start at iteration 1
    bad = compose.compose([str(ROOT / "configs" / "train")], "train_synthetic",
                          ["common.exp_name=r2", *TINY, "optimization.acc_steps=0"], apply_env=False)
    with pytest.raises(AssertionError, match="acc_steps"):
        build("train_recipe", non_resolving_instantiate(bad)).validate_config()


def test_ddp_transform_on_two_gloo_ranks_matches_one_process(unique_port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(unique_port), str(ROOT / "tests" / "_mp_ddp_check.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0 and res.stdout.count("DDP_OK") == 2, res.stdout[-2000:] + res.stderr[-3000:]


def test_bench_reference_arm_without_a_gpu_says_so_and_exits_zero():
    """On a machine without a CUDA device the reference arm prints its one-line reason and exits 0 (on a GPU box it
    runs the unmodified reference; tests/test_reference_arm.py covers the parts that need no GPU)."""
    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                         capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_graft_entry_exposes_build_and_smoke():
    import importlib.util

    spec = importlib.util.spec_from_file_location("graft_entry", ROOT / "__graft_entry__.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert callable(mod.build) and callable(mod.smoke)
