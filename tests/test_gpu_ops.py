"""Numerics of the sm_100a kernels against plain PyTorch fp32 references."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _close(a, b, rtol, atol, what=""):
    """Per element: |a - b| <= atol * rms(b) + rtol * |b| (the absolute part scales with the tensor's typical size,
    the relative part with the element itself, so small elements are held to a tight bound too)."""
    a, b = a.float(), b.float()
    rms = b.pow(2).mean().sqrt().item()
    excess = (a - b).abs() - (atol * rms + rtol * b.abs())
    worst = excess.max().item()
    assert worst <= 0, f"{what}: an element misses its bound by {worst} (rms of the reference {rms})"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1000, 776, 328), (384, 1024, 2048)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    from optimus_dl_b200.ops import _lib, gemm

    torch.manual_seed(0)
    A = torch.randn((K, M) if a_mn else (M, K), device=_dev(), dtype=torch.bfloat16)
    B = torch.randn((K, N) if b_mn else (N, K), device=_dev(), dtype=torch.bfloat16)
    out = gemm.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
    ref = (A.float().t() if a_mn else A.float()) @ (B.float() if b_mn else B.float().t())
    _lib.check_status()
    _close(out, ref, 1e-2, 1e-2, "gemm")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(2440, 2056, 200), (4096, 2320, 512)])
def test_gemm_two_sm_layouts(a_mn, b_mn, M, N, K):
    """Shapes with at least 74 tiles of 256 x 256 run on the paired-CTA kernel; ragged edges in M, N and K."""
    from optimus_dl_b200.ops import _lib, gemm

    assert ((M + 255) // 256) * ((N + 255) // 256) >= gemm.PAIR_MIN_TILES and gemm.USE_2SM
    torch.manual_seed(1)
    A = torch.randn((K, M) if a_mn else (M, K), device=_dev(), dtype=torch.bfloat16)
    B = torch.randn((K, N) if b_mn else (N, K), device=_dev(), dtype=torch.bfloat16)
    out = gemm.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
    ref = (A.float().t() if a_mn else A.float()) @ (B.float() if b_mn else B.float().t())
    _lib.check_status()
    _close(out, ref, 1e-2, 1e-2, "two-SM gemm")
    again = gemm.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
    assert torch.equal(out, again), "the paired kernel must be deterministic"


def test_gemm_two_sm_epilogues_and_swiglu():
    from optimus_dl_b200.ops import _lib, gemm

    torch.manual_seed(2)
    M, N, K = 2304, 2312, 320
    A = torch.randn(M, K, device=_dev(), dtype=torch.bfloat16)
    B = torch.randn(N, K, device=_dev(), dtype=torch.bfloat16)
    bias = torch.randn(N, device=_dev(), dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    _close(gemm.gemm(A, B, out_dtype=torch.float32), ref, 1e-5, 1e-3, "fp32 out")
    acc = torch.ones(M, N, device=_dev(), dtype=torch.float32)
    gemm.gemm(A, B, out=acc, accumulate=True)
    _close(acc, ref + 1.0, 1e-5, 1e-3, "accumulate fp32")
    accb = torch.ones(M, N, device=_dev(), dtype=torch.bfloat16)
    gemm.gemm(A, B, out=accb, accumulate=True)
    _close(accb, ref + 1.0, 1e-2, 1e-2, "accumulate bf16")
    _close(gemm.gemm(A, B, bias=bias, act="silu", alpha=0.05), torch.nn.functional.silu(ref * 0.05 + bias.float()), 1e-2, 1e-2,
           "bias+silu")
    d, f, T = 320, 1160, 2304            # 9 x 10 tiles of 256 rows x 128 output columns
    x = (torch.randn(T, d, device=_dev()) * 0.5).to(torch.bfloat16)
    w1 = (torch.randn(f, d, device=_dev()) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(f, d, device=_dev()) * 0.05).to(torch.bfloat16)
    h, g, u = gemm.swiglu_gemm(x, w1, w2)
    gr, ur = x.float() @ w1.float().t(), x.float() @ w2.float().t()
    _close(g, gr, 1e-2, 1e-2, "gate")
    _close(u, ur, 1e-2, 1e-2, "up")
    _close(h, torch.nn.functional.silu(gr) * ur, 2e-2, 2e-2, "h")
    _lib.check_status()


@pytest.mark.parametrize("softcap", [(0, 1.0), (1, 30.0), (2, 1.0)])
def test_cross_entropy_statistics_from_the_gemm_epilogue(softcap, monkeypatch):
    """Per-row (max, sum-exp, sum, target logit, arg-max) straight from the accumulator tiles against the statistics
    kernel on materialised bf16 logits; vocabulary not a multiple of the tile, targets outside the slice, rows not
    a multiple of the tile; then the whole loss without gradients against the same call with gradients."""
    from optimus_dl_b200.ops import _lib, gemm
    from optimus_dl_b200.ops.cross_entropy import linear_cross_entropy

    monkeypatch.setattr(gemm, "CE_STATS_MIN_K", 0)     # the dispatch keeps small K on the two-kernel path
    torch.manual_seed(13)
    mode, cap = softcap
    rows, d, V, off = 2304 + 24, 328, 2312 + 56, 1000
    x = (torch.randn(rows, d, device=_dev()) * 0.7).bfloat16()
    w = (torch.randn(V, d, device=_dev()) * 0.2).bfloat16()
    tg = torch.randint(0, V + 2 * off, (rows,), device=_dev(), dtype=torch.int64)      # some fall outside [off, off + V)
    tg[::7] = -100
    st = torch.empty(5, rows, device=_dev(), dtype=torch.float32)
    bi = torch.empty(rows, device=_dev(), dtype=torch.int32)
    assert gemm.ce_stats_gemm(x, w, tg, st, bi, off, mode, cap)
    logits = gemm.gemm(x, w)
    st_r = torch.empty_like(st)
    bi_r = torch.empty_like(bi)
    l = _lib.lib()
    _lib.check(l.ob_ce_stats(_lib.ptr(logits), logits.stride(0), _lib.ptr(tg), _lib.ptr(st_r[0]), _lib.ptr(st_r[1]),
                             _lib.ptr(st_r[2]), _lib.ptr(st_r[3]), _lib.ptr(st_r[4]), _lib.ptr(bi_r), rows, V, off, mode, cap,
                             _lib.stream()), "ob_ce_stats")
    assert torch.equal(st[0], st_r[0]) and torch.equal(st[4], st_r[4]) and torch.equal(st[3], st_r[3])
    assert torch.equal(bi, bi_r)
    lse, lse_r = st[0] + st[1].log(), st_r[0] + st_r[1].log()
    assert (lse - lse_r).abs().max().item() < 1e-4
    assert ((st[2] - st_r[2]).abs() <= 1e-4 * st_r[2].abs() + 2e-2).all()
    _lib.check_status()

    tg2 = torch.randint(0, V, (rows,), device=_dev(), dtype=torch.int64)
    tg2[::5] = -100
    kw = dict(label_smoothing=0.1, softcap=cap if mode == 1 else None, softcap_type="sigmoid" if mode == 2 else "tanh")
    with torch.no_grad():
        a = linear_cross_entropy(x, w, tg2, **kw)
    xg = x.clone().requires_grad_(True)
    b = linear_cross_entropy(xg, w, tg2, **kw)
    assert abs(a.loss.item() - b.loss.item()) < 1e-4 * max(1.0, abs(b.loss.item()))
    assert a.n_correct.item() == b.n_correct.item() and a.n_valid.item() == b.n_valid.item()
    _lib.check_status()


def test_swiglu_backward_fused_into_the_down_projection_gradient():
    """dh = dy Wc never reaches memory: the GEMM epilogue reads g / u and leaves dg / du in their place. Checked
    against the fp32 formulas, with a ragged last tile in both directions."""
    from optimus_dl_b200.ops import _lib, gemm

    torch.manual_seed(11)
    T, D, F = 2304 + 40, 328, 2312           # more than 74 tiles of 256 x 256; T, F not multiples of the tile
    dy = (torch.randn(T, D, device=_dev()) * 0.5).bfloat16()
    wc = (torch.randn(D, F, device=_dev()) * 0.05).bfloat16()
    g = torch.randn(T, F, device=_dev()).bfloat16()
    u = torch.randn(T, F, device=_dev()).bfloat16()
    g0, u0 = g.float(), u.float()
    assert gemm.swiglu_bwd_gemm(dy, wc, g, u)
    dh = (dy.float() @ wc.float()).bfloat16().float()
    sg = torch.sigmoid(g0)
    _close(g, dh * u0 * sg * (1 + g0 * (1 - sg)), 2e-2, 2e-2, "dg")
    _close(u, dh * g0 * sg, 2e-2, 2e-2, "du")
    _lib.check_status()


@pytest.mark.parametrize("layout", ["fwd", "dgrad", "wgrad"])
def test_gemm_at_flagship_shapes(layout):
    """The MLP products of the 8B config at full size (8192 tokens, 4096 x 14336), in the three operand layouts of
    a linear layer, checked on sampled rows against fp32."""
    from optimus_dl_b200.ops import _lib, gemm

    torch.manual_seed(5)
    T, D, F = 8192, 4096, 14336
    if layout == "fwd":        # h[T,F] W[D,F]^T
        a = torch.randn(T, F, device=_dev()).bfloat16()
        b = (torch.randn(D, F, device=_dev()) * 0.05).bfloat16()
        out = gemm.gemm(a, b)
        rows = torch.randint(0, T, (96,), device=_dev())
        ref = a[rows].float() @ b.float().t()
    elif layout == "dgrad":    # dy[T,D] W[D,F]  (W read MN-major)
        a = torch.randn(T, D, device=_dev()).bfloat16()
        b = (torch.randn(D, F, device=_dev()) * 0.05).bfloat16()
        out = gemm.gemm(a, b, b_mn=True)
        rows = torch.randint(0, T, (96,), device=_dev())
        ref = a[rows].float() @ b.float()
    else:                      # dy[T,F]^T x[T,D]  (both MN-major, K = tokens)
        a = torch.randn(T, F, device=_dev()).bfloat16()
        b = torch.randn(T, D, device=_dev()).bfloat16()
        out = gemm.gemm(a, b, a_mn=True, b_mn=True)
        rows = torch.randint(0, F, (96,), device=_dev())
        ref = a[:, rows].float().t() @ b.float()
    torch.cuda.synchronize()
    _lib.check_status()
    _close(out[rows], ref, 1e-2, 1e-2, f"{layout} at flagship size")


@pytest.mark.parametrize("M", [1, 8, 33, 64])
@pytest.mark.parametrize("N,K", [(4104, 2048), (1000, 200), (151936, 512)])
def test_gemm_skinny_decode_shapes(M, N, K, monkeypatch):
    """At most 64 rows without gradients: the weight-streaming kernel (weight rows on the M side of the MMA, the
    reduction split over the CTAs of a cluster when there are few weight tiles), with and without bias. The size
    threshold below which the library is used is lowered so that every shape reaches the kernel."""
    from optimus_dl_b200.ops import _lib, gemm

    monkeypatch.setattr(gemm, "SKINNY_MIN_WEIGHT", 0)
    torch.manual_seed(3)
    x = torch.randn(M, K, device=_dev(), dtype=torch.bfloat16)
    w = (torch.randn(N, K, device=_dev()) * 0.1).to(torch.bfloat16)
    bias = torch.randn(N, device=_dev(), dtype=torch.bfloat16)
    before = _lib.launch_count()
    with torch.no_grad():
        y = gemm.gemm(x, w)
        yb = gemm.gemm(x, w, bias=bias)
    assert _lib.launch_count() - before == 2      # both products went through this library's launcher, not a library GEMM
    ref = x.float() @ w.float().t()
    _lib.check_status()
    _close(y, ref, 1e-2, 1e-2, "skinny")
    _close(yb, ref + bias.float(), 1e-2, 1e-2, "skinny + bias")


def test_gemm_epilogues():
    from optimus_dl_b200.ops import _lib, gemm

    torch.manual_seed(0)
    A = torch.randn(512, 256, device=_dev(), dtype=torch.bfloat16)
    B = torch.randn(384, 256, device=_dev(), dtype=torch.bfloat16)
    bias = torch.randn(384, device=_dev(), dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    out32 = gemm.gemm(A, B, out_dtype=torch.float32)
    _close(out32, ref, 1e-5, 1e-3, "fp32 out")
    acc = torch.ones(512, 384, device=_dev(), dtype=torch.float32)
    gemm.gemm(A, B, out=acc, accumulate=True)
    _close(acc, ref + 1.0, 1e-5, 1e-3, "accumulate")
    g = gemm.gemm(A, B, bias=bias, act="gelu", alpha=0.05)
    _close(g, torch.nn.functional.gelu(ref * 0.05 + bias.float()), 1e-2, 1e-2, "bias+gelu")
    _lib.check_status()


def test_swiglu_dual_gemm_and_mlp_grad():
    from optimus_dl_b200.ops import _lib, activation, gemm

    torch.manual_seed(0)
    d, f, T = 256, 768, 384
    x = (torch.randn(T, d, device=_dev()) * 0.5).to(torch.bfloat16).requires_grad_()
    w1 = (torch.randn(f, d, device=_dev()) * 0.05).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(f, d, device=_dev()) * 0.05).to(torch.bfloat16).requires_grad_()
    wc = (torch.randn(d, f, device=_dev()) * 0.05).to(torch.bfloat16).requires_grad_()
    h, g, u = gemm.swiglu_gemm(x.detach(), w1.detach(), w2.detach())
    gr, ur = x.float() @ w1.float().t(), x.float() @ w2.float().t()
    _close(g, gr, 1e-2, 1e-2, "gate")
    _close(h, torch.nn.functional.silu(gr) * ur, 2e-2, 2e-2, "h")
    y = activation.swiglu_mlp(x, w1, w2, wc)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, w1f, w2f, wcf = [t.detach().float().requires_grad_() for t in (x, w1, w2, wc)]
    yr = (torch.nn.functional.silu(xf @ w1f.t()) * (xf @ w2f.t())) @ wcf.t()
    yr.backward(dy.float())
    _close(y, yr, 2e-2, 2e-2, "mlp y")
    for a, b, n in ((x.grad, xf.grad, "dx"), (w1.grad, w1f.grad, "dw1"), (w2.grad, w2f.grad, "dw2"), (wc.grad, wcf.grad, "dwc")):
        _close(a, b, 3e-2, 3e-2, n)
    _lib.check_status()


@pytest.mark.parametrize("D", [512, 4096])
def test_rmsnorm_fwd_bwd(D):
    from optimus_dl_b200.ops import norm

    torch.manual_seed(0)
    x = torch.randn(300, D, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    res = torch.randn(300, D, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=_dev())).to(torch.bfloat16).requires_grad_()
    y, h = norm.rms_norm(x, w, 1e-5, residual=res)
    dy, dh = torch.randn_like(y), torch.randn_like(h)
    (y * dy).sum().backward(retain_graph=True)
    gx1 = x.grad.clone()
    x.grad = None; res.grad = None; w.grad = None
    torch.autograd.backward([y, h], [dy, dh])
    xf, rf, wf = [t.detach().float().requires_grad_() for t in (x, res, w)]
    hf = (xf + rf).to(torch.bfloat16).float()  # the stream is stored in bf16
    hf2 = xf + rf
    yr = hf2 * torch.rsqrt(hf2.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    torch.autograd.backward([yr, hf2], [dy.float(), dh.float()])
    _close(y, yr, 2e-2, 2e-2, "y")
    _close(h, hf, 1e-2, 1e-2, "h")
    _close(x.grad, xf.grad, 3e-2, 3e-2, "dx")
    _close(res.grad, rf.grad, 3e-2, 3e-2, "dres")
    _close(w.grad, wf.grad, 3e-2, 5e-2, "dw")
    assert gx1.isfinite().all()


def test_layernorm_fwd_bwd():
    from optimus_dl_b200.ops import norm

    torch.manual_seed(0)
    D = 768
    x = torch.randn(257, D, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=_dev())).to(torch.bfloat16).requires_grad_()
    b = (0.1 * torch.randn(D, device=_dev())).to(torch.bfloat16).requires_grad_()
    y = norm.layer_norm(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf, bf = [t.detach().float().requires_grad_() for t in (x, w, b)]
    yr = torch.nn.functional.layer_norm(xf, (D,), wf, bf, 1e-5)
    yr.backward(dy.float())
    _close(y, yr, 2e-2, 2e-2, "y")
    _close(x.grad, xf.grad, 3e-2, 3e-2, "dx")
    _close(w.grad, wf.grad, 3e-2, 5e-2, "dw")
    _close(b.grad, bf.grad, 3e-2, 5e-2, "db")


def test_adamw_matches_torch():
    from optimus_dl_b200.ops import optim

    torch.manual_seed(0)
    n = 100003
    p0 = torch.randn(n, device=_dev())
    ref = torch.nn.Parameter(p0.clone())
    o = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    master, m, v = p0.clone(), torch.zeros(n, device=_dev()), torch.zeros(n, device=_dev())
    lp = torch.empty(n, device=_dev(), dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device=_dev()).to(torch.bfloat16)
        ref.grad = g.float()
        o.step()
        optim.adamw_step_(master, m, v, g, lp, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    _close(master, ref.detach(), 1e-5, 1e-5, "adamw")
    _close(lp, ref.detach(), 1e-2, 1e-2, "bf16 copy")
    out = torch.zeros(1, device=_dev())
    optim.sumsq_(g, out)
    _close(out, g.float().pow(2).sum().reshape(1), 1e-4, 1e-3, "sumsq")


@pytest.mark.parametrize("softcap,stype,smooth", [(None, "tanh", 0.0), (30.0, "tanh", 0.1), (None, "sigmoid", 0.0)])
def test_linear_cross_entropy(softcap, stype, smooth):
    from optimus_dl_b200.ops import _lib, cross_entropy as ce

    torch.manual_seed(0)
    T, d, V = 700, 256, 5003
    x = torch.randn(T, d, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, d, device=_dev()) * 0.05).to(torch.bfloat16).requires_grad_()
    tg = torch.randint(0, V, (T,), device=_dev())
    tg[::7] = -100
    res = ce.linear_cross_entropy(x, w, tg, label_smoothing=smooth, softcap=softcap, softcap_type=stype, chunk_rows=256)
    res.loss.backward()
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logits = (xf @ wf.t())
    r = ce.cross_entropy_ref(logits.detach().to(torch.bfloat16).float() + (logits - logits.detach()), tg, -100, smooth, softcap, stype)
    r.loss.backward()
    assert abs(res.loss.item() - r.loss.item()) < 2e-2 * max(1.0, abs(r.loss.item()))
    assert int(res.n_valid) == int(r.n_valid)
    assert abs(int(res.n_correct) - int(r.n_correct)) <= 2
    _close(x.grad, xf.grad, 5e-2, 2e-2, "dx")
    _close(w.grad, wf.grad, 5e-2, 5e-2, "dw")
    _lib.check_status()


def test_embedding_fwd_bwd():
    from optimus_dl_b200.ops import embedding

    torch.manual_seed(0)
    V, D = 1000, 256
    table = torch.randn(V, D, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 50, (4, 64), device=_dev())  # many repeats
    out = embedding.embedding(ids, table)
    dout = torch.randn_like(out)
    out.backward(dout)
    tf = table.detach().float().requires_grad_()
    torch.nn.functional.embedding(ids, tf).backward(dout.float())
    assert torch.equal(out, table.detach()[ids])
    _close(table.grad, tf.grad, 2e-2, 2e-2, "dtable")


@pytest.mark.parametrize("hd,norm", [(64, False), (128, False), (128, True)])
def test_rope_kernel_matches_reference(hd, norm):
    from optimus_dl_b200.ops import rope

    torch.manual_seed(0)
    T, Hq, Hk = 100, 4, 2
    W = (Hq + 2 * Hk) * hd
    qkv = torch.randn(T, W, device=_dev(), dtype=torch.bfloat16)
    freqs = rope.precompute_freqs_cis(hd, 256, 10000.0).to(_dev())
    pos = torch.randint(0, 256, (T,), device=_dev(), dtype=torch.int32)
    qw = (1 + 0.1 * torch.randn(hd, device=_dev())).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * torch.randn(hd, device=_dev())).to(torch.bfloat16) if norm else None
    out = torch.empty_like(qkv)
    rstd = torch.empty(T, Hq + Hk, device=_dev()) if norm else None
    rope.rope_kernel_fwd(qkv, out, W, W, freqs, pos, qw, kw, rstd, T, Hq, Hk, hd, 256, 1e-6)
    q = qkv[:, : Hq * hd].view(1, T, Hq, hd)
    k = qkv[:, Hq * hd: (Hq + Hk) * hd].view(1, T, Hk, hd)
    if norm:
        from optimus_dl_b200.ops.norm import rms_norm_ref

        q, k = rms_norm_ref(q, qw, 1e-6), rms_norm_ref(k, kw, 1e-6)
    qr, kr = rope.apply_rotary_emb(q, k, freqs, pos.long().view(1, T))
    _close(out[:, : Hq * hd].view(1, T, Hq, hd), qr, 2e-2, 2e-2, "q")
    _close(out[:, Hq * hd: (Hq + Hk) * hd].view(1, T, Hk, hd), kr, 2e-2, 2e-2, "k")


def test_flag_wait_times_out():
    """A GEMM whose operand flags nobody sets must give up after its bounded wait, report it through the status
    word and leave the context usable (no trap, no hang)."""
    import time

    from optimus_dl_b200.ops import _lib, gemm

    dev = torch.device("cuda")
    a = torch.randn(128, 128, device=dev).bfloat16()
    b = torch.randn(256, 128, device=dev).bfloat16()
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    t0 = time.time()
    gemm.gemm(a, b, b_flags=flags, flag_rows=128, flag_value=1, tile_order=1)
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.0 < waited < 20.0, waited
    with pytest.raises(_lib.KernelError, match="flag wait timed out"):
        _lib.check_status(dev)
    _lib.check_status(dev)   # the status word was cleared by the report
    # the same operation with the flags set completes and is correct
    flags.fill_(1)
    out = gemm.gemm(a, b, b_flags=flags, flag_rows=128, flag_value=1, tile_order=1)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    ref = a.float() @ b.float().t()
    assert (out.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item()
