"""SwiGLU: ``h = silu(g) * u`` (elementwise kernels in ``csrc/elementwise.cu``) and the fused
dual-GEMM form ``h = silu(x W1^T) * (x W2^T)`` whose epilogue never writes ``g`` and ``u``
twice (``csrc/gemm_core.cuh``). Replaces Liger's SwiGLU used by the reference at
optimus_dl/modules/model/blocks/mlp.py:73-78.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib, gemm


def _ok(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and ts[0].numel() % 8 == 0


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g = g.contiguous()
        u = u.contiguous()
        h = torch.empty_like(g)
        _lib.check(_lib.lib().ob_swiglu_fwd(_lib.ptr(g), _lib.ptr(u), _lib.ptr(h), g.numel(), _lib.stream()), "swiglu_fwd")
        ctx.save_for_backward(g, u)
        return h

    @staticmethod
    def backward(ctx, dh):
        g, u = ctx.saved_tensors
        dh = dh.contiguous()
        dg = torch.empty_like(g)
        du = torch.empty_like(u)
        _lib.check(_lib.lib().ob_swiglu_bwd(_lib.ptr(dh), _lib.ptr(g), _lib.ptr(u), _lib.ptr(dg), _lib.ptr(du), None,
                                            g.numel(), _lib.stream()), "swiglu_bwd")
        return dg, du


def swiglu_backward(dh: torch.Tensor, g: torch.Tensor, u: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(dg, du)`` of ``h = silu(g) * u`` (no autograd; kernel on CUDA bf16)."""
    if _ok(dh, g, u):
        dg = torch.empty_like(g)
        du = torch.empty_like(u)
        _lib.check(_lib.lib().ob_swiglu_bwd(_lib.ptr(dh), _lib.ptr(g), _lib.ptr(u), _lib.ptr(dg), _lib.ptr(du), None,
                                            g.numel(), _lib.stream()), "swiglu_bwd")
        return dg, du
    gf, uf, df = g.float(), u.float(), dh.float()
    sig = torch.sigmoid(gf)
    dg = df * uf * sig * (1.0 + gf * (1.0 - sig))
    du = df * gf * sig
    return dg.to(g.dtype), du.to(u.dtype)


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """``silu(g) * u`` with autograd."""
    if _ok(g, u):
        return _SwiGLU.apply(g, u)
    return F.silu(g) * u


class _SwiGLUMLPUp(torch.autograd.Function):
    """``h = silu(x W1^T) * (x W2^T)`` in one GEMM launch; saves g and u for the backward."""

    @staticmethod
    def forward(ctx, x, w1, w2):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        h, g, u = gemm.swiglu_gemm(x2, w1, w2, save_gu=True)
        ctx.save_for_backward(x2, w1, w2, g, u)
        ctx.params = (w1, w2)
        return h.view(*shp[:-1], w1.shape[0])

    @staticmethod
    def backward(ctx, dh):
        x2, w1, w2, g, u = ctx.saved_tensors
        dh2 = dh.reshape(-1, dh.shape[-1]).contiguous()
        dg = torch.empty_like(g)
        du = torch.empty_like(u)
        _lib.check(_lib.lib().ob_swiglu_bwd(_lib.ptr(dh2), _lib.ptr(g), _lib.ptr(u), _lib.ptr(dg), _lib.ptr(du), None,
                                            g.numel(), _lib.stream()), "swiglu_bwd")
        dx = dw1 = dw2 = None
        if ctx.needs_input_grad[0]:
            dx = gemm.gemm(dg, w1, b_mn=True)
            gemm.gemm(du, w2, b_mn=True, out=dx, accumulate=True)
            dx = dx.view(*dh.shape[:-1], x2.shape[-1])
        from .linear import main_grad_of, main_grad_write

        for i, (p, d) in enumerate(zip(ctx.params, (dg, du))):
            if not ctx.needs_input_grad[1 + i]:
                continue
            mg = main_grad_of(p)
            if mg is not None:
                gemm.gemm(d, x2, a_mn=True, b_mn=True, out=mg, accumulate=main_grad_write(p))
            elif i == 0:
                dw1 = gemm.gemm(d, x2, a_mn=True, b_mn=True)
            else:
                dw2 = gemm.gemm(d, x2, a_mn=True, b_mn=True)
        return dx, dw1, dw2


def swiglu_mlp_up(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """Gate/up projections and SwiGLU; dual-B tcgen05 GEMM on CUDA bf16, eager otherwise."""
    if _ok(x, w1, w2) and w1.shape == w2.shape and w1.stride() == w2.stride():
        return _SwiGLUMLPUp.apply(x, w1, w2)
    return F.silu(F.linear(x, w1)) * F.linear(x, w2)


class _SwiGLUMLP(torch.autograd.Function):
    """Whole SwiGLU feed-forward ``(silu(x W1^T) * (x W2^T)) Wc^T``.

    Saves only ``x``, ``g`` and ``u``: the product ``h`` that feeds the down projection is rebuilt
    by the backward activation kernel (it is needed there for the down projection's weight
    gradient), which removes one ``[tokens, hidden]`` tensor per layer from the saved set.
    """

    @staticmethod
    def forward(ctx, x, w1, w2, wc):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        h, g, u = gemm.swiglu_gemm(x2, w1, w2, save_gu=True)
        y = gemm.gemm(h, wc)
        ctx.save_for_backward(x2, w1, w2, wc, g, u)
        ctx.params = (w1, w2, wc)
        return y.view(*shp[:-1], wc.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .linear import main_grad_of, main_grad_write

        x2, w1, w2, wc, g, u = ctx.saved_tensors
        p1, p2, pc = ctx.params
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dh = gemm.gemm(dy2, wc, b_mn=True)
        h = torch.empty_like(g)
        # in place: g <- dg, u <- du (the saved tensors are dead after this call)
        _lib.check(_lib.lib().ob_swiglu_bwd(_lib.ptr(dh), _lib.ptr(g), _lib.ptr(u), _lib.ptr(g), _lib.ptr(u), _lib.ptr(h),
                                            g.numel(), _lib.stream()), "swiglu_bwd")
        dg, du = g, u
        del dh
        grads = [None, None, None]
        for i, (p, a, b) in enumerate(((pc, dy2, h), (p1, dg, x2), (p2, du, x2))):
            if not ctx.needs_input_grad[(3, 1, 2)[i]]:
                continue
            mg = main_grad_of(p)
            if mg is not None:
                gemm.gemm(a, b, a_mn=True, b_mn=True, out=mg, accumulate=main_grad_write(p))
            else:
                grads[i] = gemm.gemm(a, b, a_mn=True, b_mn=True)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm.gemm(dg, w1, b_mn=True)
            gemm.gemm(du, w2, b_mn=True, out=dx, accumulate=True)
            dx = dx.view(*dy.shape[:-1], x2.shape[-1])
        return dx, grads[1], grads[2], grads[0]


def swiglu_mlp(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, wc: torch.Tensor) -> torch.Tensor:
    """Bias-free SwiGLU feed-forward block; kernels on CUDA bf16, eager otherwise."""
    if _ok(x, w1, w2, wc) and not torch.is_grad_enabled() and x.numel() // x.shape[-1] <= gemm.SKINNY_M:
        # decode steps: weight-streaming products (see gemm.gemm) and the elementwise activation
        from . import linear as lin_ops

        gu = lin_ops.multi_linear(x, [w1, w2])
        g, u = gu.split(w1.shape[0], dim=-1)
        return lin_ops.linear(swiglu(g.contiguous(), u.contiguous()), wc)
    if _ok(x, w1, w2, wc) and w1.shape == w2.shape and w1.stride() == w2.stride() and wc.shape[1] % 8 == 0:
        return _SwiGLUMLP.apply(x, w1, w2, wc)
    return F.linear(F.silu(F.linear(x, w1)) * F.linear(x, w2), wc)
