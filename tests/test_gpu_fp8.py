"""Block-scaled e4m3 GEMM, quantisers and the FP8 linear path against fp32 PyTorch statements."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dq_row(q, s):
    rows, cols = q.shape
    return (q.float().view(rows, cols // 128, 128) * s.t()[:, :, None]).view(rows, cols)


def test_rowwise_quantiser():
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    x = (torch.randn(300, 512, device="cuda") * torch.rand(300, 1, device="cuda") * 4).bfloat16()
    x[5] = 0
    q, s = fp8.quantize_rowwise(x)
    qr, sr = fp8.quantize_rowwise_ref(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (4, 300)
    assert torch.allclose(s, sr, rtol=1e-6)
    assert (q.float() == qr.float()).float().mean() > 0.999
    rel = (_dq_row(q, s) - x.float()).abs().max() / x.float().abs().max()
    assert rel < 0.07
    assert torch.all(_dq_row(q, s)[5] == 0)


def test_block_quantiser_and_transpose():
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    w = (torch.randn(400, 384, device="cuda") * 0.05).bfloat16()
    q, s, qt, st = fp8.quantize_block(w, with_transpose=True)
    qr, sr = fp8.quantize_block_ref(w)
    assert s.shape == (4, 3) and st.shape == (3, 4)
    assert torch.allclose(s, sr, rtol=1e-6) and torch.equal(st, s.t())
    assert (q.float() == qr.float()).float().mean() > 0.999
    assert torch.equal(qt.float(), q.float().t())


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (512, 1024, 1024), (300, 400, 384), (4096, 4096, 4096), (77, 130, 256)])
def test_fp8_gemm_matches_dequantised_product(M, N, K):
    from optimus_dl_b200.ops import _lib, fp8

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    a8, sa = fp8.quantize_rowwise_ref(a)
    b8, sb = fp8.quantize_block_ref(b)
    out = fp8.gemm_fp8(a8, sa, b8, sb)
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda"))
    ref = fp8.gemm_fp8_ref(a8, sa, b8, sb)
    err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-9)
    assert err < 1e-2, err
    # and the whole chain is a usable approximation of the bf16 product
    exact = a.float() @ b.float().t()
    rel = (out.float() - exact).norm() / exact.norm()
    assert rel < 0.06, rel


def test_fp8_linear_forward_backward():
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    x = torch.randn(2, 192, 512, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(768, device="cuda").bfloat16().requires_grad_(True)
    y = fp8.fp8_linear(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xf, wf, bf)
    yr.backward(dy.float())
    rel = lambda a, r: ((a.float() - r).norm() / r.norm()).item()  # noqa: E731
    assert rel(y, yr) < 0.05
    assert rel(x.grad, xf.grad) < 0.06
    assert rel(w.grad, wf.grad) < 0.02     # weight gradient stays in bf16
    assert rel(b.grad, bf.grad) < 0.02
    # the cache follows the parameter version
    first = w._fp8_cache[0]
    with torch.no_grad():
        w.add_(0.01)
    fp8.fp8_linear(x, w, b)
    assert w._fp8_cache[0] != first


def test_fp8_training_tracks_bf16():
    from optimus_dl_b200.amp.fp8 import FP8Recipe
    from optimus_dl_b200.criterion.cross_entropy import CrossEntropyCriterion, CrossEntropyCriterionConfig
    from optimus_dl_b200.model_transforms.transformer_engine import mark_fp8_linears
    from optimus_dl_b200.models.llama2 import Llama, LlamaConfig

    def run(fp8_on: bool):
        torch.manual_seed(0)
        cfg = LlamaConfig(n_layer=2, n_head=4, n_kv_head=2, n_embd=256, vocab_size=512, sequence_length=128,
                          intermediate_size=512, tie_word_embeddings=False)
        model = Llama(cfg).to(device="cuda", dtype=torch.bfloat16)
        if fp8_on:
            assert mark_fp8_linears(model) == 14
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
        crit = CrossEntropyCriterion(CrossEntropyCriterionConfig())
        recipe = FP8Recipe()
        ids = torch.randint(0, 512, (4, 129), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
        losses = []
        for _ in range(12):
            opt.zero_grad()
            with recipe.autocast(fp8_on):
                loss, _ = crit(model, {"input_ids": ids})
                loss.backward()
            opt.step()
            losses.append(loss.item())
        return losses

    ref, got = run(False), run(True)
    assert got[-1] < got[0] - 0.5, got
    assert abs(got[-1] - ref[-1]) < 0.25, (ref[-1], got[-1])
    assert abs(got[0] - ref[0]) < 0.05


def test_tensor_quantiser_and_scale():
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    x = (torch.randn(300, 520, device="cuda") * 3).bfloat16()
    q, s = fp8.quantize_tensor(x)
    qr, sr = fp8.quantize_tensor_ref(x)
    assert s.shape == (1,) and torch.allclose(s, sr, rtol=1e-6)
    assert (q.float() == qr.float()).float().mean() > 0.999
    # the workspace is left clean: a second tensor gets its own maximum
    y = (x * 0.01).bfloat16()
    _, s2 = fp8.quantize_tensor(y)
    assert torch.allclose(s2, y.float().abs().amax().reshape(1) / 448.0, rtol=1e-6)
    # given scale + recorded maximum
    rec = torch.zeros(1, dtype=torch.int32, device="cuda")
    q3, _ = fp8.quantize_tensor(x, scale=s, amax_rec=rec)
    assert torch.equal(q3.float(), q.float())
    assert rec.view(torch.float32).item() == x.float().abs().max().item()
    z = torch.zeros(16, 64, device="cuda", dtype=torch.bfloat16)
    assert fp8.quantize_tensor(z)[1].item() == 1.0


def test_weight_tensor_quantiser_transpose():
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    w = (torch.randn(400, 384, device="cuda") * 0.05).bfloat16()
    q, s, qt = fp8.quantize_weight_tensor(w)
    qr, sr = fp8.quantize_tensor_ref(w)
    assert torch.allclose(s, sr, rtol=1e-6)
    assert (q.float() == qr.float()).float().mean() > 0.999
    assert torch.equal(qt.float(), q.float().t())


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (512, 1024, 1024), (300, 400, 384), (4096, 4096, 4096), (77, 130, 256)])
def test_fp8_tensor_gemm(M, N, K):
    from optimus_dl_b200.ops import _lib, fp8

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    a8, sa = fp8.quantize_tensor_ref(a)
    b8, sb = fp8.quantize_tensor_ref(b)
    out = fp8.gemm_fp8_tensor(a8, sa, b8, sb)
    torch.cuda.synchronize()
    _lib.check_status(torch.device("cuda"))
    ref = fp8.gemm_fp8_tensor_ref(a8, sa, b8, sb)
    err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-9)
    assert err < 1e-2, err
    exact = a.float() @ b.float().t()
    assert (out.float() - exact).norm() / exact.norm() < 0.07


@pytest.mark.parametrize("kind", ["tensorwise", "delayed"])
def test_fp8_linear_per_tensor_recipes(kind):
    from optimus_dl_b200.amp.fp8 import FP8Recipe, Fp8Format, parse_fp8_recipe
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    recipe = FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe(kind), amax_history_len=4)
    x = torch.randn(2, 192, 512, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    xf, wf = (t.detach().float().requires_grad_(True) for t in (x, w))
    rel = lambda a, r: ((a.float() - r).norm() / r.norm()).item()  # noqa: E731
    for step in range(3):
        x.grad = w.grad = xf.grad = wf.grad = None
        with recipe.backward(True):
            assert fp8.scaling_mode() == ("tensor" if kind == "tensorwise" else "delayed")
            y = fp8.fp8_linear(x, w)
            # shrinking magnitudes: a delayed scale never saturates on them (growth would, by design)
            dy = torch.randn_like(y) * (1.0 - 0.2 * step)
            y.backward(dy)
        yr = torch.nn.functional.linear(xf, wf)
        yr.backward(dy.float())
        assert rel(y, yr) < 0.06, (step, rel(y, yr))
        assert rel(x.grad, xf.grad) < 0.07, (step, rel(x.grad, xf.grad))
        assert rel(w.grad, wf.grad) < 0.06     # per-tensor recipes also run the weight gradient in FP8
    if kind == "delayed":
        ds = recipe.delayed_state
        assert len(ds.rows) == 2 and ds.pos == 3
        st = ds.state[:2].cpu()
        assert (st[:, 1] == 0).all()                     # recorded maxima were consumed
        assert (st[:, 2:5] > 0).all()                    # three history entries filled
        assert torch.allclose(st[:, 0], st[:, 2:].amax(1) / 448.0)


def test_fp8_training_per_tensor_tracks_bf16():
    from optimus_dl_b200.amp.fp8 import FP8Recipe, Fp8Format, parse_fp8_recipe
    from optimus_dl_b200.criterion.cross_entropy import CrossEntropyCriterion, CrossEntropyCriterionConfig
    from optimus_dl_b200.model_transforms.transformer_engine import mark_fp8_linears
    from optimus_dl_b200.models.llama2 import Llama, LlamaConfig

    def run(kind):
        torch.manual_seed(0)
        cfg = LlamaConfig(n_layer=2, n_head=4, n_kv_head=2, n_embd=256, vocab_size=512, sequence_length=128,
                          intermediate_size=512, tie_word_embeddings=False)
        model = Llama(cfg).to(device="cuda", dtype=torch.bfloat16)
        if kind:
            mark_fp8_linears(model)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
        crit = CrossEntropyCriterion(CrossEntropyCriterionConfig())
        recipe = FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe(kind or "blockwise"))
        ids = torch.randint(0, 512, (4, 129), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
        losses = []
        for _ in range(12):
            opt.zero_grad()
            with recipe.backward(bool(kind)):
                loss, _ = crit(model, {"input_ids": ids})
                loss.backward()
            opt.step()
            losses.append(loss.item())
        return losses

    ref = run(None)
    for kind in ("tensorwise", "delayed"):
        got = run(kind)
        assert got[-1] < got[0] - 0.5, (kind, got)
        assert abs(got[-1] - ref[-1]) < 0.3, (kind, ref[-1], got[-1])


def test_fp8_tensor_gemm_accumulates():
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    a = torch.randn(256, 384, device="cuda").bfloat16()
    b = torch.randn(200, 384, device="cuda").bfloat16()
    a8, sa = fp8.quantize_tensor(a)
    b8, sb = fp8.quantize_tensor(b)
    base = torch.randn(256, 200, device="cuda").bfloat16()
    out = base.clone()
    fp8.gemm_fp8_tensor(a8, sa, b8, sb, out=out, accumulate=True)
    ref = base.float() + fp8.gemm_fp8_tensor_ref(a8, sa, b8, sb)
    assert (out.float() - ref).abs().max() / ref.abs().max() < 1e-2


def test_fp8_wgrad_path_and_main_grad():
    from optimus_dl_b200.amp.fp8 import FP8Recipe, Fp8Format, parse_fp8_recipe
    from optimus_dl_b200.ops import fp8

    torch.manual_seed(0)
    rel = lambda a, r: ((a.float() - r).norm() / r.norm()).item()  # noqa: E731
    x = torch.randn(2, 128, 512, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(768, 512, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    w.main_grad = torch.zeros_like(w)
    w._main_grad_filled = False
    xf, wf = (t.detach().float().requires_grad_(True) for t in (x, w))
    with FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe("tensorwise")).backward(True):
        for _ in range(2):                      # second pass accumulates into main_grad
            y = fp8.fp8_linear(x, w)
            assert y.grad_fn is not None
            dy = torch.randn_like(y)
            y.backward(dy)
            torch.nn.functional.linear(xf, wf).backward(dy.float())
    assert w.grad is None and w._main_grad_filled
    assert rel(w.main_grad, wf.grad) < 0.06, rel(w.main_grad, wf.grad)
    assert rel(x.grad, xf.grad) < 0.07
    # wgrad=False keeps the weight gradient in bf16
    w2 = w.detach().clone().requires_grad_(True)
    with FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe("tensorwise"), wgrad=False).backward(True):
        assert not fp8.fp8_wgrad_enabled()
        y = fp8.fp8_linear(x.detach(), w2)
        y.backward(dy)
    wr = wf.detach().clone().requires_grad_(True)
    torch.nn.functional.linear(xf.detach(), wr).backward(dy.float())
    assert rel(w2.grad, wr.grad) < 0.02


def test_rmsnorm_emits_block_quantised_output():
    from optimus_dl_b200.amp.fp8 import FP8Recipe
    from optimus_dl_b200.model_transforms.transformer_engine import mark_fp8_linears, mark_fp8_norms
    from optimus_dl_b200.models.llama2 import Llama, LlamaConfig
    from optimus_dl_b200.ops import fp8, norm

    torch.manual_seed(0)
    for D in (512, 2048, 4096):
        x = torch.randn(3, 100, D, device="cuda").bfloat16()
        r = torch.randn_like(x)
        w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
        y0, h0 = norm.rms_norm(x, w, 1e-5, r)
        y, h = norm.rms_norm(x, w, 1e-5, r, emit_fp8=True)
        assert torch.equal(y, y0) and torch.equal(h, h0)
        q, s = y._fp8_rowwise
        qr, sr = fp8.quantize_rowwise(y0)
        assert q.shape == (300, D) and torch.equal(s, sr)
        assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
        assert fp8.quantize_rowwise(y)[0] is q          # the consumer takes the attached form
    # in a model: same losses with and without the fused quantiser, gradients flow
    def run(fuse):
        torch.manual_seed(0)
        cfg = LlamaConfig(n_layer=2, n_head=4, n_kv_head=2, n_embd=256, vocab_size=512, sequence_length=128,
                          intermediate_size=512, tie_word_embeddings=False)
        model = Llama(cfg).to(device="cuda", dtype=torch.bfloat16)
        mark_fp8_linears(model)
        if fuse:
            assert mark_fp8_norms(model) == 4
        ids = torch.randint(0, 512, (4, 128), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
        with FP8Recipe().autocast(True):
            out = model(ids)["logits"].float()
            loss = out.logsumexp(-1).mean()
            loss.backward()
        return loss.item(), model.transformer.h[0].ln_1.weight.grad.float().norm().item()

    a, b = run(False), run(True)
    assert abs(a[0] - b[0]) < 1e-3 and abs(a[1] - b[1]) / a[1] < 1e-2, (a, b)
