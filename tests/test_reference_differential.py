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
@pytest.mark.parametrize("check", ["models", "train_parts", "data", "checkpoints", "recipe", "recipe_accumulation", "recipe_resume", "pretokenize", "generation", "metrics_recipe", "eval_adapter"])
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
    the lm_eval adapter's scores in its reference-scoring mode."""
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_ref_diff_worker.py"), check], capture_output=True,
                         text=True, timeout=900, env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT))
    assert res.returncode == 0 and f"DIFF_OK {check}" in res.stdout, res.stdout[-1500:] + res.stderr[-3000:]
