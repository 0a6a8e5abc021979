"""The reference arm of bench.py: the tree under baseline/_ref is the upstream package, byte for byte, and it
imports and trains with the stand-in third-party modules, in a process that never imports this package."""

import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
import reference_arm  # noqa: E402

UPSTREAM = "/root/reference/optimus_dl"


def _have_tree() -> bool:
    return reference_arm.ensure_reference_tree() and reference_arm.reference_root() is not None


@pytest.mark.skipif(not os.path.isdir(UPSTREAM), reason="no upstream checkout on this machine")
def test_reference_tree_is_unmodified():
    assert _have_tree()
    mine = os.path.join(reference_arm.reference_root(), "optimus_dl")
    assert reference_arm.tree_digest(mine) == reference_arm.tree_digest(UPSTREAM)


@pytest.mark.skipif(not _have_tree(), reason="reference tree not present")
def test_reference_builds_and_steps_without_this_package():
    code = textwrap.dedent(f"""
        import sys
        sys.path.insert(0, {os.path.join(ROOT, 'baseline', '_ref')!r}); sys.path.insert(0, {os.path.join(ROOT, 'baseline', 'ref_deps')!r})
        import logging; logging.disable(logging.INFO)
        import torch, optimus_dl
        from optimus_dl.modules.criterion import build_criterion
        from optimus_dl.modules.distributed import build_best_collective
        from optimus_dl.modules.distributed.config import DistributedConfig
        from optimus_dl.modules.optim import build_optimizer
        from optimus_dl.recipe.mixins.model_builder import ModelBuilder, ModelBuilderConfig
        col = build_best_collective(DistributedConfig(tp_size=1, sharding_world_size=1), torch.device("cpu"))
        cfg = dict(_name="llama2", n_layer=2, n_head=8, n_kv_head=2, n_embd=128, intermediate_size=256, vocab_size=512,
                   rope_theta=500000.0, sequence_length=64, tie_word_embeddings=False)
        tr = [{{"_name": "activation_checkpoint", "layer_classes": ["LlamaBlock"]}},
              {{"_name": "fully_shard", "reshard_after_forward": False,
                "mixed_precision": {{"param_dtype": "bfloat16", "reduce_dtype": "float32"}}}}]
        m = ModelBuilder(ModelBuilderConfig(), model_transforms=tr).build_model(dict(cfg), collective=col)
        assert type(m).__module__ == "optimus_dl.modules.model.llama2"
        crit = build_criterion({{"_name": "cross_entropy"}}, collective=col)
        opt = build_optimizer({{"_name": "adamw", "lr": 1e-3, "betas": [0.9, 0.95], "fused": False}}, params=m.make_parameter_groups())
        ids = torch.randint(0, 512, (2, 33)); losses = []
        for _ in range(4):
            opt.zero_grad()
            with torch.autocast("cpu", dtype=torch.bfloat16):
                loss, _ = crit(m, {{"input_ids": ids}})
            loss.backward(); opt.step(); losses.append(float(loss))
        assert losses[-1] < losses[0], losses
        assert not any(k.startswith("optimus_dl_b200") for k in sys.modules)
        print("ok")
    """)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
