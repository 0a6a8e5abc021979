"""Differential tests against the unmodified reference: the upstream package (the tree the reference arm of bench.py
runs, with stand-ins for the third-party modules this image lacks) and this package are loaded into one CPU process
and fed the same inputs. Skipped where that tree is not present."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
import reference_arm  # noqa: E402


def _have_tree() -> bool:
    return reference_arm.ensure_reference_tree() and reference_arm.reference_root() is not None


@pytest.mark.skipif(not _have_tree(), reason="reference tree not present")
@pytest.mark.parametrize("check", ["models", "train_parts", "data", "checkpoints", "recipe", "recipe_accumulation", "recipe_resume", "pretokenize", "generation", "metrics_recipe", "eval_adapter", "schedules", "optimizer_routing"])
def test_same_inputs_give_the_same_results_as_the_reference(check):
    """``models``: logits and parameter groups of every model family from shared weights, plain and packed batches;
    ``train_parts``: criterion loss and meters, AdamW and SOAP under every schedule; ``data``: identical batches and
    resumption from each other's state for four pipelines on one and three ranks; ``checkpoints``: save with one
    manager, load with the other, continue bit-identically, both directions; ``recipe``: the whole training recipe,
    every logged number of every iteration; ``recipe_accumulation``: the same with two accumulation steps, gradient
    clipping and bf16 autocast (1e-3: autocast rounds in a slightly different order); ``recipe_resume``: four iterations,
    then a second run that resumes from the checkpoint and continues to eight; ``pretokenize``: the data-preparation
    recipe writes byte-identical shards and the same index; ``generation``: greedy and seeded sampled decoding give
    the same tokens; ``metrics_recipe``: the metrics recipe's results and log records; ``eval_adapter``:
    the lm_eval adapter's scores in its reference-scoring mode; ``schedules``: every learning-rate schedule, step by step;
    ``optimizer_routing``: which parameters Muon's and a composite's sub-optimizers get."""
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_ref_diff_worker.py"), check], capture_output=True,
                         text=True, timeout=900, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT))
    assert res.returncode == 0 and f"DIFF_OK {check}" in res.stdout, res.stdout[-1500:] + res.stderr[-3000:]


@pytest.mark.skipif(not _have_tree(), reason="reference tree not present")
def test_two_rank_ddp_recipe_logs_the_same_numbers_as_the_reference(tmp_path, unique_port):
    """The training recipe on two Gloo ranks with the ``ddp`` transform, each code base under its own ``torchrun``:
    per-rank data shares, gradient averaging and the cross-rank aggregation of meters give the same log records."""
    worker = os.path.join(ROOT, "tests", "_ref_diff_worker.py")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
    import socket

    for side in ("ref", "ours"):
        port = unique_port
        if side == "ours":                         # a second free port for the second launch
            with socket.socket() as s:
                s.bind(("127.0.0.1", 0))
                port = s.getsockname()[1]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
               "--master-port", str(port), worker, "recipe_ddp_side", side, str(tmp_path)]
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        assert res.returncode == 0 and res.stdout.count("DIFF_OK") == 2, res.stdout[-1500:] + res.stderr[-3000:]
    res = subprocess.run([sys.executable, worker, "recipe_ddp_side", "compare", str(tmp_path)], capture_output=True, text=True,
                         timeout=300, env=env)
    assert res.returncode == 0 and "DIFF_OK" in res.stdout, res.stdout[-1500:] + res.stderr[-3000:]
