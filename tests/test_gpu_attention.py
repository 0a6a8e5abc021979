"""tcgen05 attention kernels against the fp32 masked-softmax reference."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_fwd(q, k, v, doc_start, window, scale):
    from optimus_dl_b200.ops import _lib

    N, Hq, hd = q.shape
    Hk = k.shape[1]
    out = torch.empty(N, Hq * hd, device=q.device, dtype=torch.bfloat16)
    lse = torch.empty(Hq, N, device=q.device, dtype=torch.float32)
    rc = _lib.lib().ob_attn_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(doc_start),
                                N, Hq, Hk, hd, q.stride(0), k.stride(0), out.stride(0), float(scale), int(window or 0),
                                _lib.ptr(_lib.status_word(q.device)), _lib.stream())
    assert rc == 0
    torch.cuda.synchronize()
    _lib.check_status()
    return out.view(N, Hq, hd), lse


def _docs(N, lens, device):
    ids = torch.cat([torch.full((l,), i) for i, l in enumerate(lens)])[:N]
    from optimus_dl_b200.ops.attention import build_doc_start

    return build_doc_start(1, N, device, document_ids=ids.view(1, N).to(device))


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("N,lens,window", [(256, None, None), (1000, None, None), (777, [100, 333, 5, 339], None),
                                           (1024, [512, 512], 200), (640, None, 128)])
def test_attention_forward(hd, N, lens, window):
    from optimus_dl_b200.ops.attention import attention_ref, build_doc_start

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    Hq, Hk = 4, 2
    qkv = torch.randn(N, (Hq + 2 * Hk) * hd, device=dev, dtype=torch.bfloat16)
    q = qkv[:, : Hq * hd].view(N, Hq, hd)
    k = qkv[:, Hq * hd: (Hq + Hk) * hd].view(N, Hk, hd)
    v = qkv[:, (Hq + Hk) * hd:].view(N, Hk, hd)
    ds = _docs(N, lens, dev) if lens else build_doc_start(1, N, dev)
    scale = 1.0 / math.sqrt(hd)
    out, lse = _run_fwd(q, k, v, ds, window, scale)
    ref = attention_ref(q, k, v, ds, window, scale)
    err = (out.float() - ref.float()).abs().max().item()
    assert err < 3e-2, f"max err {err}"


@pytest.mark.parametrize("hd,use_norm", [(128, False), (64, False), (128, True)])
@pytest.mark.parametrize("N,lens,window", [(256, None, None), (900, [100, 333, 5, 462], None), (640, None, 128)])
def test_qkv_attention_forward_backward(hd, use_norm, N, lens, window):
    """Fused QK-norm + RoPE + attention (kernels) versus the PyTorch path on fp32 copies."""
    from optimus_dl_b200.ops import _lib
    from optimus_dl_b200.ops.attention import build_doc_start, qkv_attention
    from optimus_dl_b200.ops.rope import precompute_freqs_cis

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    Hq, Hk = 4, 2
    W = (Hq + 2 * Hk) * hd
    base = torch.randn(1, N, W, device=dev) * 0.7
    ds = _docs(N, lens, dev) if lens else build_doc_start(1, N, dev)
    freqs = precompute_freqs_cis(hd, 1024, 10000.0).to(dev)
    qw = (1 + 0.1 * torch.randn(hd, device=dev)) if use_norm else None
    kw = (1 + 0.1 * torch.randn(hd, device=dev)) if use_norm else None
    dy = torch.randn(1, N, Hq * hd, device=dev)

    def run(dtype):
        x = base.to(dtype).detach().clone().requires_grad_()
        a = qw.to(dtype).detach().clone().requires_grad_() if use_norm else None
        b = kw.to(dtype).detach().clone().requires_grad_() if use_norm else None
        # the kernel path rotates its input in place: hand it a private copy that autograd tracks
        y = qkv_attention(x * 1.0, n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=ds, freqs_cis=freqs,
                          q_norm_weight=a, k_norm_weight=b, norm_eps=1e-6, window=window)
        y.backward(dy.to(dtype))
        return y, x.grad, (a.grad if use_norm else None), (b.grad if use_norm else None)

    y_k, dx_k, da_k, db_k = run(torch.bfloat16)
    torch.cuda.synchronize()
    _lib.check_status()
    y_r, dx_r, da_r, db_r = run(torch.float32)

    def rel(a, b):
        return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)

    assert rel(y_k, y_r) < 3e-2, rel(y_k, y_r)
    assert rel(dx_k, dx_r) < 5e-2, rel(dx_k, dx_r)
    if use_norm:
        assert rel(da_k, da_r) < 8e-2 and rel(db_k, db_r) < 8e-2, (rel(da_k, da_r), rel(db_k, db_r))


def _exp_doc_lengths(total, seed=0, mean=2048, lo=32):
    g = torch.Generator().manual_seed(seed)
    lens, n = [], 0
    while n < total:
        l = max(lo, int(torch.empty(1).exponential_(1.0 / mean, generator=g).item()))
        lens.append(min(l, total - n))
        n += lens[-1]
    return lens


@pytest.mark.parametrize("T,Hq,Hk,packed", [(8192, 32, 8, False), (8192, 32, 8, True), (16384, 40, 8, True)])
def test_attention_at_flagship_shapes(T, Hq, Hk, packed):
    """Full sequence lengths of the benchmark configs (hundreds of key tiles, document boundaries inside 128-row
    tiles at large offsets): forward and backward of the kernels against an fp32 masked-softmax reference evaluated
    completely for the query heads of two key/value groups."""
    from optimus_dl_b200.ops import _lib
    from optimus_dl_b200.ops.attention import build_doc_start, mask_from_doc_start, qkv_attention

    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    hd, G = 128, Hq // Hk
    qkv = (torch.randn(1, T, (Hq + 2 * Hk) * hd, device=dev) * 0.7).bfloat16().requires_grad_(True)
    ds = _docs(T, _exp_doc_lengths(T), dev) if packed else build_doc_start(1, T, dev)
    dout = torch.randn(1, T, Hq * hd, device=dev).bfloat16()
    out = qkv_attention(qkv, n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=ds)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_status()
    dqkv = qkv.grad[0]
    scale = 1.0 / math.sqrt(hd)
    mask = mask_from_doc_start(ds)
    flat = qkv.detach()[0]
    for kvh in (1, Hk - 1):
        kf = flat[:, (Hq + kvh) * hd:(Hq + kvh + 1) * hd].float().requires_grad_(True)
        vf = flat[:, (Hq + Hk + kvh) * hd:(Hq + Hk + kvh + 1) * hd].float().requires_grad_(True)
        for h in range(kvh * G, (kvh + 1) * G):
            qf = flat[:, h * hd:(h + 1) * hd].float().requires_grad_(True)
            s = (qf @ kf.t()) * scale
            p = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
            o = p @ vf
            del s, p
            o.backward(dout[0, :, h * hd:(h + 1) * hd].float())
            got_o = out[0, :, h * hd:(h + 1) * hd].float()
            assert (got_o - o.detach()).abs().max().item() < 3e-2, f"out head {h}"
            got_dq = dqkv[:, h * hd:(h + 1) * hd].float()
            tol = 2e-2 * qf.grad.abs().max().item() + 1e-3
            assert (got_dq - qf.grad).abs().max().item() < tol, f"dq head {h}"
            del o, qf
        for name, ref_g, off in (("dk", kf.grad, Hq + kvh), ("dv", vf.grad, Hq + Hk + kvh)):
            got = dqkv[:, off * hd:(off + 1) * hd].float()
            tol = 2e-2 * ref_g.abs().max().item() + 1e-3
            assert (got - ref_g).abs().max().item() < tol, f"{name} group {kvh}"
        del kf, vf
