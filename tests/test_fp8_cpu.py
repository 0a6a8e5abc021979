"""CPU statements of the per-tensor FP8 path and the recipe plumbing around it."""

import torch


def test_tensor_reference_round_trip():
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    a = torch.randn(64, 256).bfloat16()
    b = (torch.randn(48, 256) * 0.1).bfloat16()
    a8, sa = fp8.quantize_tensor_ref(a)
    b8, sb = fp8.quantize_tensor_ref(b)
    assert sa.shape == (1,) and abs(sa.item() - a.float().abs().max().item() / 448.0) < 1e-6
    out = fp8.gemm_fp8_tensor(a8, sa, b8, sb)          # CPU: falls back to the fp32 statement
    exact = a.float() @ b.float().t()
    assert out.dtype == torch.bfloat16
    assert (out.float() - exact).norm() / exact.norm() < 0.07
    q, s, qt = fp8.quantize_weight_tensor(b)
    assert torch.equal(qt.float(), q.float().t()) and torch.equal(s, sb)


def test_recipe_selects_scaling_mode():
    from optimus_dl_b200.amp.fp8 import FP8Recipe, Fp8Format, Fp8RecipeType, parse_fp8_recipe
    from optimus_dl_b200.ops import fp8

    assert fp8.scaling_mode() == "block"
    for name, mode in (("blockwise", "block"), ("mxfp8", "block"), ("current", "tensor"), ("delayed", "delayed")):
        r = FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe(name), margin=1)
        with r.autocast(True):
            assert fp8.scaling_mode() == mode
            assert fp8._margin_mul() == 2.0
        assert fp8.scaling_mode() == "block"
    d = FP8Recipe(Fp8Format.E4M3, Fp8RecipeType.DELAYED, amax_history_len=8, amax_compute_algo="most_recent")
    assert d.delayed_state.H == 8 and not d.delayed_state.use_max
    with d.backward(True):        # no state yet: the update on exit is a no-op
        pass
    assert d.delayed_state.pos == 0


def test_reference_call_forms_of_the_fp8_helpers(monkeypatch):
    from optimus_dl_b200.amp import fp8 as A

    assert A.get_fp8_format_from_string("Hybrid") is A.Fp8Format.HYBRID
    assert A.get_fp8_recipe_type_from_string("MXFP8") is A.Fp8RecipeType.MXFP8
    assert A.get_transformer_engine_version() is None or isinstance(A.get_transformer_engine_version(), str)
    assert A.create_fp8_recipe("delayed", "hybrid") is None            # no CUDA device here
    monkeypatch.setattr(A.torch.cuda, "is_available", lambda: True)
    r = A.create_fp8_recipe("delayed", "e4m3", margin=2, amax_history_len=8, amax_compute_algo="most_recent")
    assert r.recipe is A.Fp8RecipeType.DELAYED and r.format is A.Fp8Format.E4M3 and r.options["margin"] == 2
    assert r.delayed_state.H == 8 and not r.delayed_state.use_max
    r = A.create_fp8_recipe(A.Fp8RecipeConfig(recipe_type="tensorwise"))
    assert r.recipe is A.Fp8RecipeType.TENSORWISE and r.delayed_state is None
    r = A.create_fp8_recipe({"enabled": True, "recipe": "blockwise", "wgrad": False})
    assert r.recipe is A.Fp8RecipeType.BLOCKWISE and r.options["wgrad"] is False
    assert A.create_fp8_recipe({"enabled": False, "recipe": "blockwise"}) is None


_REDUCE_WORKER = '''
import os, sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
from optimus_dl_b200.ops.fp8 import reduce_recorded_maxima
dist.init_process_group("gloo")
r = dist.get_rank()
state = torch.zeros(4, 2 + 3)
state[:, 0] = 9.0                                   # scales are not touched
state[:3, 1] = torch.tensor([1.0, 5.0, 0.0]) if r == 0 else torch.tensor([4.0, 2.0, 0.5])
state[3, 1] = 100.0 + r                             # beyond n_rows: left alone
reduce_recorded_maxima(state, 3)
assert state[:3, 1].tolist() == [4.0, 5.0, 0.5], state
assert state[3, 1].item() == 100.0 + r and (state[:, 0] == 9.0).all()
reduce_recorded_maxima(state, 0)
dist.barrier()
print("REDUCE_OK", r)
dist.destroy_process_group()
'''


def test_recorded_maxima_are_reduced_over_ranks(tmp_path, unique_port):
    import os
    import subprocess
    import sys

    from optimus_dl_b200.ops.fp8 import reduce_recorded_maxima

    lone = torch.tensor([[1.0, 3.0, 0.0]])
    reduce_recorded_maxima(lone, 1)                     # no process group: nothing happens
    assert lone.tolist() == [[1.0, 3.0, 0.0]]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "w.py"
    script.write_text(_REDUCE_WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(unique_port), str(script), root]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0 and res.stdout.count("REDUCE_OK") == 2, res.stdout[-2000:] + res.stderr[-3000:]


def test_training_context_entries_follow_the_reference_contract():
    """``TrainingContextMixin(optimization_config).setup_training_context(device)``: the scaler is always a
    ``GradScaler`` (disabled on CPU and with FP8), the two context entries can be entered directly or called, and
    an fp8 dtype without ``fp8.enabled`` runs bf16 autocast
    (optimus_dl/recipe/train/mixins/execution/context_mixin.py:42-150)."""
    import contextlib

    import torch

    from optimus_dl_b200.amp.config import AmpConfig, Fp8Config, OptimizationConfig
    from optimus_dl_b200.recipe.train.mixins.execution.context_mixin import FreshContext, TrainingContextMixin

    mixin = TrainingContextMixin(OptimizationConfig(amp=AmpConfig(enabled=True, dtype="torch.bfloat16", enable_scaler=True)))
    ctx = mixin.setup_training_context(torch.device("cpu"))
    assert isinstance(ctx["scaler"], torch.GradScaler) and not ctx["scaler"].is_enabled()
    assert ctx["fp8_recipe"] is None and ctx["fp8_enabled"] is False and ctx["is_fp8_dtype"] is False
    assert isinstance(ctx["amp_ctx"], FreshContext) and isinstance(mixin.get_fp8_backward_ctx(), contextlib.nullcontext)
    a = torch.randn(4, 4)
    with ctx["amp_ctx"]:
        assert (a @ a).dtype == torch.bfloat16
        with ctx["amp_ctx"]():                      # nested, through the call form
            assert (a @ a).dtype == torch.bfloat16
    assert (a @ a).dtype == torch.float32
    with ctx["fp8_backward_ctx"], ctx["fp8_backward_ctx"]():
        pass
    off = TrainingContextMixin(OptimizationConfig(amp=AmpConfig(
        enabled=True, dtype="torch.float8_e4m3fn", fp8=Fp8Config(enabled=False)))).setup_training_context(torch.device("cpu"))
    assert off["is_fp8_dtype"] is True and off["fp8_enabled"] is False and off["fp8_recipe"] is None
    with off["amp_ctx"]:
        assert (a @ a).dtype == torch.bfloat16
    plain = TrainingContextMixin(OptimizationConfig(amp=AmpConfig(enabled=False))).setup_training_context(torch.device("cpu"))
    with plain["amp_ctx"]:
        assert (a @ a).dtype == torch.float32
