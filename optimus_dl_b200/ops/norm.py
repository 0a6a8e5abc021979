"""RMSNorm / LayerNorm with fp32 statistics (kernels in ``csrc/norm.cu``).

CUDA bf16 tensors run the hand-written kernels; everything else (CPU, fp32) runs the
PyTorch reference below, which is also the oracle of the numerics tests.
Math: optimus_dl/modules/model/blocks/layer_norms.py:21-120 in the reference.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


def rms_norm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)


def _kernel_ok(x: torch.Tensor) -> bool:
    D = x.shape[-1]
    return x.is_cuda and x.dtype == torch.bfloat16 and D % 8 == 0 and D <= 8192


def _bf16(t: torch.Tensor | None) -> torch.Tensor | None:
    if t is None:
        return None
    return t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps, emit_fp8=False):
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D).contiguous()
        rows = x2.shape[0]
        res2 = residual.reshape(-1, D).contiguous() if residual is not None else None
        w = _bf16(weight).contiguous()
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if res2 is not None else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        q = scales = None
        if emit_fp8 and D % 128 == 0:
            # the consumer is an FP8 linear layer: its 1x128-quantised input comes out of this launch
            q = torch.empty((rows, D), dtype=torch.float8_e4m3fn, device=x.device)
            scales = torch.empty((D // 128, rows), dtype=torch.float32, device=x.device)
            rc = _lib.lib().ob_rmsnorm_fwd_fp8(_lib.ptr(x2), _lib.ptr(res2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(h),
                                               _lib.ptr(rstd), _lib.ptr(q), _lib.ptr(scales), rows, rows, D, float(eps),
                                               _lib.stream())
            _lib.check(rc, "ob_rmsnorm_fwd_fp8")
        else:
            rc = _lib.lib().ob_rmsnorm_fwd(_lib.ptr(x2), _lib.ptr(res2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(h),
                                           _lib.ptr(rstd), rows, D, float(eps), _lib.stream())
            _lib.check(rc, "ob_rmsnorm_fwd")
        ctx.save_for_backward(h if h is not None else x2, w, rstd)
        ctx.has_res = residual is not None
        ctx.wdtype = weight.dtype
        ctx.shape = shp
        yv = y.view(shp)
        if q is not None:
            yv._fp8_rowwise = (q, scales)   # picked up by ops.fp8.quantize_rowwise
        if h is not None:
            return yv, h.view(shp)
        return yv, None

    @staticmethod
    def backward(ctx, dy, dh):
        xin, w, rstd = ctx.saved_tensors
        rows, D = xin.shape
        dy2 = dy.reshape(-1, D).contiguous()
        dres = dh.reshape(-1, D).contiguous() if (ctx.has_res and dh is not None) else None
        dx = torch.empty_like(xin)
        l = _lib.lib()
        grid = l.ob_norm_bwd_grid(rows)
        partial = torch.empty((grid, D), dtype=torch.float32, device=xin.device)
        dw = torch.empty(D, dtype=torch.bfloat16, device=xin.device)
        rc = l.ob_rmsnorm_bwd(_lib.ptr(dy2), _lib.ptr(xin), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx),
                              _lib.ptr(partial), _lib.ptr(dw), None, 0, rows, D, _lib.stream())
        _lib.check(rc, "ob_rmsnorm_bwd")
        dxv = dx.view(ctx.shape)
        return dxv, dw.to(ctx.wdtype), (dxv if ctx.has_res else None), None, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None,
             emit_fp8: bool = False):
    """``y = rmsnorm(x + residual) * weight``. Returns ``y`` or ``(y, x + residual)`` when a residual is given.
    ``emit_fp8``: also produce the 1x128 block-quantised e4m3 form of ``y`` in the same launch and attach it to
    ``y`` (``y._fp8_rowwise``) for the FP8 linear layer that consumes it."""
    if _kernel_ok(x) and (residual is None or (residual.dtype == x.dtype and residual.shape == x.shape)):
        y, h = _RMSNorm.apply(x, weight, residual, eps, emit_fp8)
        return y if residual is None else (y, h)
    if residual is not None:
        h = x + residual
        return rms_norm_ref(h, weight, eps), h
    return rms_norm_ref(x, weight, eps)


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        shp = x.shape
        D = shp[-1]
        x2 = x.reshape(-1, D).contiguous()
        rows = x2.shape[0]
        w = _bf16(weight).contiguous()
        b = _bf16(bias).contiguous() if bias is not None else None
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        rc = _lib.lib().ob_layernorm_fwd(_lib.ptr(x2), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), _lib.ptr(mean),
                                         _lib.ptr(rstd), rows, D, float(eps), _lib.stream())
        _lib.check(rc, "ob_layernorm_fwd")
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.has_bias = bias is not None
        ctx.wdtype = weight.dtype
        ctx.shape = shp
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, D = x2.shape
        dy2 = dy.reshape(-1, D).contiguous()
        l = _lib.lib()
        grid = l.ob_norm_bwd_grid(rows)
        partial = torch.empty((2 * grid, D), dtype=torch.float32, device=x2.device)
        dx = torch.empty_like(x2)
        dw = torch.empty(D, dtype=torch.bfloat16, device=x2.device)
        db = torch.empty(D, dtype=torch.bfloat16, device=x2.device)
        rc = l.ob_layernorm_bwd(_lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(w), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(dx),
                                _lib.ptr(partial), _lib.ptr(dw), _lib.ptr(db), rows, D, _lib.stream())
        _lib.check(rc, "ob_layernorm_bwd")
        return dx.view(ctx.shape), dw.to(ctx.wdtype), (db.to(ctx.wdtype) if ctx.has_bias else None), None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float = 1e-5) -> torch.Tensor:
    if _kernel_ok(x):
        return _LayerNorm.apply(x, weight, bias, eps)
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)
