"""e4m3 matrix products with block or per-tensor scales (``csrc/gemm_fp8.cu``).

Scaling follows the fine-grained scheme used for FP8 training of large models: activations (and
output gradients) carry one scale per ``1 x 128`` block along the reduction dimension, weights one
scale per ``128 x 128`` block; products accumulate in fp32 per 128-wide k-block, are scaled and
summed in registers, and leave the kernel in bf16. This is the path the reference reaches through
Transformer Engine's ``Float8BlockScaling`` recipe (optimus_dl/modules/amp/fp8.py:180-315); here it is
a hand-written tcgen05 kernel.

Per-tensor scaling (the reference's ``tensorwise`` = TE ``Float8CurrentScaling`` and ``delayed`` =
TE ``DelayedScaling`` recipes) uses one fp32 scale per operand: the tensor core then accumulates over
the whole reduction dimension in TMEM and the kernel runs at the plain e4m3 rate. ``tensorwise`` takes
the scale from the tensor's own maximum (one extra read pass); ``delayed`` takes it from a history of
maxima recorded by the quantiser in earlier steps, so quantising is a single pass.

``fp8_linear`` is the autograd function behind FP8 linear layers: forward ``y = q(x) q(W)^T`` and
input gradient ``dx = q(dy) q(W^T)^T`` in FP8, weight gradient ``dW = dy^T x`` in bf16 (it feeds the
fp32 master-weight update and is the product most sensitive to quantisation noise). The quantised
weight and its transpose are cached per parameter version, i.e. re-made once per optimizer step.
"""

from __future__ import annotations

from typing import Any

import torch

from . import _lib, gemm
from . import linear as lin_ops

E4M3_MAX = 448.0
BLOCK = 128


def kernel_ok(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and _lib.available()


# ---------------------------------------------------------------------- reference (PyTorch) quantisers
def quantize_rowwise_ref(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``x [rows, cols]`` -> (e4m3 values ``[rows, cols]``, scales ``[cols / 128, rows]`` fp32)."""
    rows, cols = x.shape
    xb = x.float().view(rows, cols // BLOCK, BLOCK)
    amax = xb.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xb / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(rows, cols)
    return q, scale.t().contiguous()


def quantize_block_ref(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``w [rows, cols]`` -> (e4m3 ``[rows, cols]``, scales ``[ceil(rows/128), ceil(cols/128)]``)."""
    rows, cols = w.shape
    pr, pc = (-rows) % BLOCK, (-cols) % BLOCK
    wp = torch.nn.functional.pad(w.float(), (0, pc, 0, pr))
    R, C = wp.shape[0] // BLOCK, wp.shape[1] // BLOCK
    wb = wp.view(R, BLOCK, C, BLOCK)
    amax = wb.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (wb / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).view(wp.shape)[:rows, :cols]
    return q.to(torch.float8_e4m3fn).contiguous(), scale


def gemm_fp8_ref(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """fp32 statement of the block-scaled product (dequantise, then multiply)."""
    M, K = a8.shape
    N = b8.shape[0]
    a = a8.float().view(M, K // BLOCK, BLOCK) * sa.t()[:, :, None]
    nb = torch.arange(N, device=b8.device) // BLOCK
    b = b8.float().view(N, K // BLOCK, BLOCK) * sb[nb][:, :, None]
    return a.reshape(M, K) @ b.reshape(N, K).t()


# ---------------------------------------------------------------------- kernels
def quantize_rowwise(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    pre = getattr(x, "_fp8_rowwise", None)   # left by a producer that quantised in its own launch (RMSNorm)
    if pre is not None and pre[0].shape[-1] == x.shape[-1] and pre[0].numel() == x.numel():
        return pre
    x = x.reshape(-1, x.shape[-1])
    rows, cols = x.shape
    if not kernel_ok(x) or cols % BLOCK != 0:
        return quantize_rowwise_ref(x)
    if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty((cols // BLOCK, rows), dtype=torch.float32, device=x.device)
    rc = _lib.lib().ob_quant_fp8_rowwise(_lib.ptr(x), x.stride(0), _lib.ptr(q), cols, _lib.ptr(scales), rows, rows, cols,
                                         _lib.stream())
    _lib.check(rc, "ob_quant_fp8_rowwise")
    return q, scales


def quantize_block(w: torch.Tensor, with_transpose: bool = False):
    """Returns ``(q, scales)`` or, with ``with_transpose``, ``(q, scales, q_t, scales_t)``."""
    rows, cols = w.shape
    if not kernel_ok(w) or rows % 16 != 0 or cols % 16 != 0 or not w.is_contiguous():
        q, s = quantize_block_ref(w)
        if with_transpose:
            return q, s, q.t().contiguous(), s.t().contiguous()
        return q, s
    R, C = (rows + BLOCK - 1) // BLOCK, (cols + BLOCK - 1) // BLOCK
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((R, C), dtype=torch.float32, device=w.device)
    qt = st = None
    if with_transpose:
        qt = torch.empty((cols, rows), dtype=torch.float8_e4m3fn, device=w.device)
        st = torch.empty((C, R), dtype=torch.float32, device=w.device)
    rc = _lib.lib().ob_quant_fp8_block(_lib.ptr(w), w.stride(0), _lib.ptr(q), cols, _lib.ptr(qt), rows, _lib.ptr(s),
                                       _lib.ptr(st), rows, cols, _lib.ptr(None), _lib.ptr(None), _lib.stream())
    _lib.check(rc, "ob_quant_fp8_block")
    return (q, s, qt, st) if with_transpose else (q, s)


def gemm_fp8(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor,
             out: torch.Tensor | None = None) -> torch.Tensor:
    """``C[M,N] = sum_kb sa[kb, m] sb[n // 128, kb] (A8[m, kb] . B8[n, kb])`` in bf16."""
    M, K = a8.shape
    N = b8.shape[0]
    if not (a8.is_cuda and _lib.available()) or K % BLOCK != 0 or K % 16 != 0:
        r = gemm_fp8_ref(a8, sa, b8, sb).to(torch.bfloat16)
        if out is not None:
            out.copy_(r)
            return out
        return r
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
    rc = _lib.lib().ob_gemm_fp8_block(_lib.ptr(a8), a8.stride(0), _lib.ptr(sa), sa.stride(0), _lib.ptr(b8), b8.stride(0),
                                      _lib.ptr(sb), _lib.ptr(out), out.stride(0), M, N, K,
                                      _lib.ptr(_lib.status_word(a8.device)), _lib.stream())
    _lib.check(rc, "ob_gemm_fp8_block")
    return out


# ---------------------------------------------------------------------- per-tensor scaling
def scaling_mode() -> str:
    """``block`` | ``tensor`` | ``delayed``: how the active recipe scales operands (``block`` outside a recipe)."""
    from ..amp import fp8 as amp_fp8

    rec = amp_fp8._state.get("recipe")
    kind = getattr(getattr(rec, "recipe", None), "value", "blockwise")
    return {"tensorwise": "tensor", "delayed": "delayed"}.get(kind, "block")


def _margin_mul() -> float:
    from ..amp import fp8 as amp_fp8

    rec = amp_fp8._state.get("recipe")
    return float(2.0 ** int((getattr(rec, "options", None) or {}).get("margin", 0) or 0))


def quantize_tensor_ref(x: torch.Tensor, scale: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``x`` -> (e4m3 values, fp32 scale ``[1]``) with one scale for the whole tensor."""
    if scale is None:
        amax = x.float().abs().amax()
        scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax)).reshape(1)
    q = (x.float() / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, scale


def gemm_fp8_tensor_ref(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    return (a8.float() @ b8.float().t()) * (sa.float() * sb.float())


_workspaces: dict = {}


def _amax_ws(device: torch.device) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(2, dtype=torch.int32, device=device)
        _workspaces[key] = ws
    return ws


def _rows_ok(x: torch.Tensor) -> torch.Tensor:
    if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    return x


def tensor_scale(x: torch.Tensor, out: torch.Tensor | None = None, margin_mul: float = 1.0) -> torch.Tensor:
    """fp32 ``[1]``: ``max|x| / 448 * margin_mul`` (1 for an all-zero tensor), computed on the device."""
    x = _rows_ok(x.reshape(-1, x.shape[-1]))
    out = out if out is not None else torch.empty(1, dtype=torch.float32, device=x.device)
    rc = _lib.lib().ob_fp8_amax_scale(_lib.ptr(x), x.stride(0), x.shape[0], x.shape[1], _lib.ptr(_amax_ws(x.device)),
                                      _lib.ptr(out), float(margin_mul), _lib.stream())
    _lib.check(rc, "ob_fp8_amax_scale")
    return out


def quantize_tensor(x: torch.Tensor, scale: torch.Tensor | None = None, amax_rec: torch.Tensor | None = None,
                    margin_mul: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """``x [rows, cols]`` -> (e4m3 ``[rows, cols]``, scale ``[1]``). With ``scale`` given the tensor is read once;
    ``amax_rec`` (one 32-bit word) receives the running ``max|x|`` for a delayed-scaling history."""
    x = x.reshape(-1, x.shape[-1])
    rows, cols = x.shape
    if not kernel_ok(x) or cols % 8 != 0:
        return quantize_tensor_ref(x, scale)
    x = _rows_ok(x)
    if scale is None:
        scale = tensor_scale(x, margin_mul=margin_mul)
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    rc = _lib.lib().ob_quant_fp8_tensor(_lib.ptr(x), x.stride(0), _lib.ptr(q), cols, _lib.ptr(scale), _lib.ptr(amax_rec),
                                        rows, cols, _lib.stream())
    _lib.check(rc, "ob_quant_fp8_tensor")
    return q, scale


def quantize_tensor_t(w: torch.Tensor, scale: torch.Tensor | None = None, amax_rec: torch.Tensor | None = None,
                      margin_mul: float = 1.0) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``w [rows, cols]`` -> (e4m3 ``w``, scale ``[1]``, e4m3 ``w^T``) with one scale for the matrix: both
    layouts from one read of ``w`` (weights for forward / dgrad; activations and output gradients for
    forward-or-dgrad / wgrad)."""
    rows, cols = w.shape
    if not kernel_ok(w) or rows % 16 != 0 or cols % 16 != 0:
        q, s = quantize_tensor_ref(w, scale)
        return q, s, q.t().contiguous()
    w = _rows_ok(w)
    s = scale if scale is not None else tensor_scale(w, margin_mul=margin_mul)
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=w.device)
    qt = torch.empty((cols, rows), dtype=torch.float8_e4m3fn, device=w.device)
    rc = _lib.lib().ob_quant_fp8_tensor_t(_lib.ptr(w), w.stride(0), _lib.ptr(q), cols, _lib.ptr(qt), rows, _lib.ptr(s),
                                          _lib.ptr(amax_rec), rows, cols, _lib.stream())
    _lib.check(rc, "ob_quant_fp8_tensor_t")
    return q, s, qt


def quantize_weight_tensor(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return quantize_tensor_t(w)


def gemm_fp8_tensor(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor,
                    out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """``C[M,N] (+)= sa * sb * (A8 . B8^T)`` in bf16; ``sa`` / ``sb`` are fp32 ``[1]`` tensors on the device."""
    M, K = a8.shape
    N = b8.shape[0]
    assert not accumulate or out is not None
    if not (a8.is_cuda and _lib.available()) or K % BLOCK != 0 or a8.stride(0) % 16 != 0 or b8.stride(0) % 16 != 0:
        r = gemm_fp8_tensor_ref(a8, sa, b8, sb)
        if out is not None:
            out.copy_(out.float() + r if accumulate else r)
            return out
        return r.to(torch.bfloat16)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a8.device)
    rc = _lib.lib().ob_gemm_fp8_tensor(_lib.ptr(a8), a8.stride(0), _lib.ptr(sa), _lib.ptr(b8), b8.stride(0), _lib.ptr(sb),
                                       _lib.ptr(out), out.stride(0), M, N, K, int(accumulate),
                                       _lib.ptr(_lib.status_word(a8.device)), _lib.stream())
    _lib.check(rc, "ob_gemm_fp8_tensor")
    return out


def reduce_recorded_maxima(state: torch.Tensor, n_rows: int, group: Any = None) -> None:
    """Maximum over the ranks of ``group`` (default: all ranks) of the recorded ``max|x|`` column of the first
    ``n_rows`` state rows, in place: every rank then derives the same scales (the reference's ``reduce_amax``).
    Every rank must call it with the same ``n_rows``; a no-op without an initialised multi-rank process group."""
    import torch.distributed as dist

    if n_rows <= 0 or not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    col = state[:n_rows, 1].contiguous()       # non-negative floats: their maximum is the maximum of the bit patterns
    dist.all_reduce(col, op=dist.ReduceOp.MAX, group=group)
    state[:n_rows, 1].copy_(col)


class DelayedScaling:
    """Amax histories for the ``delayed`` recipe: one row ``[scale, recorded max, hist[H]]`` per (weight, role).

    A row is created on first use and seeded with the tensor's own maximum (so the first step behaves like
    current scaling); afterwards quantising uses the stored scale and records the maximum it saw, and
    :meth:`update` (once per backward pass) rolls every history and refreshes every scale with one launch.
    """

    def __init__(self, history: int = 16, algo: str = "max", capacity: int = 1024, reduce_amax: bool = True):
        self.H, self.use_max, self.capacity = max(1, int(history)), algo != "most_recent", capacity
        self.reduce_amax = bool(reduce_amax)
        self.state: torch.Tensor | None = None
        self.rows: dict = {}
        self.pos = 0

    def row(self, holder: torch.Tensor, role: str, x: torch.Tensor, margin_mul: float) -> tuple[torch.Tensor, torch.Tensor]:
        """``(scale [1], amax word [1])`` views for this tensor role, seeded from ``x`` on first use."""
        if self.state is None:
            self.state = torch.zeros((self.capacity, 2 + self.H), dtype=torch.float32, device=x.device)
        key = (id(holder), role)
        i = self.rows.get(key)
        fresh = i is None
        if fresh:
            i = len(self.rows)
            if i >= self.capacity:
                raise RuntimeError("delayed-scaling state is full; raise DelayedScaling(capacity=...)")
            self.rows[key] = i
        st = self.state[i]
        if fresh:
            tensor_scale(x, out=st[0:1], margin_mul=margin_mul)
        return st[0:1], st[1:2]

    def update(self, margin_mul: float = 1.0, group: Any = None) -> None:
        if self.state is None or not self.rows:
            return
        if self.reduce_amax:
            reduce_recorded_maxima(self.state, len(self.rows), group)
        rc = _lib.lib().ob_fp8_delayed_update(_lib.ptr(self.state), len(self.rows), self.H, self.pos, float(margin_mul),
                                              int(self.use_max), _lib.stream())
        _lib.check(rc, "ob_fp8_delayed_update")
        self.pos = (self.pos + 1) % self.H


def _delayed() -> "DelayedScaling | None":
    from ..amp import fp8 as amp_fp8

    rec = amp_fp8._state.get("recipe")
    return getattr(rec, "delayed_state", None)


def _quantize_activation(x2: torch.Tensor, holder: torch.Tensor, role: str) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor quantisation of an activation / output gradient under the active recipe."""
    mm = _margin_mul()
    ds = _delayed() if scaling_mode() == "delayed" else None
    if ds is None or not kernel_ok(x2):
        return quantize_tensor(x2, margin_mul=mm)
    scale, rec = ds.row(holder, role, x2, mm)
    return quantize_tensor(x2, scale=scale, amax_rec=rec)


def _quantize_activation_t(x2: torch.Tensor, holder: torch.Tensor, role: str):
    """Like :func:`_quantize_activation` but also returns the transposed e4m3 copy (for the wgrad product)."""
    mm = _margin_mul()
    ds = _delayed() if scaling_mode() == "delayed" else None
    if ds is None or not kernel_ok(x2):
        return quantize_tensor_t(x2, margin_mul=mm)
    scale, rec = ds.row(holder, role, x2, mm)
    return quantize_tensor_t(x2, scale=scale, amax_rec=rec)


def fp8_wgrad_enabled() -> bool:
    """Weight gradients in FP8 too: per-tensor recipes unless the recipe was built with ``wgrad=False``."""
    from ..amp import fp8 as amp_fp8

    rec = amp_fp8._state.get("recipe")
    return scaling_mode() != "block" and bool((getattr(rec, "options", None) or {}).get("wgrad", True))


def _cached_weight_tensor(w: torch.Tensor, holder: torch.Tensor | None = None):
    holder = holder if holder is not None else w
    key = (w.data_ptr(), holder._version, tuple(w.shape), _weights_epoch)
    hit = getattr(holder, "_fp8_cache_t", None)
    if hit is None or hit[0] != key:
        hit = (key, *quantize_weight_tensor(w.detach()))
        holder._fp8_cache_t = hit
    return hit[1:]


# ---------------------------------------------------------------------- autograd
_weights_epoch = 0


def weights_changed() -> None:
    """Invalidate every cached quantised weight. Called by optimizers that update parameters through raw
    pointers (the fused reduce-scatter + AdamW kernel), where the autograd version counter does not move."""
    global _weights_epoch
    _weights_epoch += 1


def _cached_weight(w: torch.Tensor, holder: torch.Tensor | None = None):
    """Quantised weight and transpose, re-made when the parameter's version counter moves. ``holder`` is
    the long-lived tensor the cache is attached to when ``w`` is a temporary view of several parameters."""
    holder = holder if holder is not None else w
    key = (w.data_ptr(), holder._version, tuple(w.shape), _weights_epoch)
    hit = getattr(holder, "_fp8_cache", None)
    if hit is None or hit[0] != key:
        q, s, qt, st = quantize_block(w.detach(), with_transpose=True)
        hit = (key, q, s, qt, st)
        holder._fp8_cache = hit
    return hit[1:]


def _fwd(x2: torch.Tensor, w: torch.Tensor, holder: torch.Tensor) -> torch.Tensor:
    if scaling_mode() == "block":
        wq, ws, _, _ = _cached_weight(w, holder)
        xq, xs = quantize_rowwise(x2)
        return gemm_fp8(xq, xs, wq, ws)
    wq, ws, _ = _cached_weight_tensor(w, holder)
    xq, xs = _quantize_activation(x2, holder, "x")
    return gemm_fp8_tensor(xq, xs, wq, ws)


def _dgrad(dy2: torch.Tensor, w: torch.Tensor, holder: torch.Tensor) -> torch.Tensor:
    if scaling_mode() == "block":
        _, _, wqt, wst = _cached_weight(w, holder)
        dq, ds = quantize_rowwise(dy2)
        return gemm_fp8(dq, ds, wqt, wst)
    _, ws, wqt = _cached_weight_tensor(w, holder)
    dq, ds = _quantize_activation(dy2, holder, "dy")
    return gemm_fp8_tensor(dq, ds, wqt, ws)


def forward_product(x2: torch.Tensor, owners: list[torch.Tensor]) -> torch.Tensor:
    """``x2 @ cat(owners)^T`` with both operands quantised (no autograd); ``owners`` adjacent or single."""
    w = owners[0] if len(owners) == 1 else lin_ops._fused_view(list(owners))
    return _fwd(x2, w, owners[0])


def dgrad_product(dy2: torch.Tensor, owners: list[torch.Tensor]) -> torch.Tensor:
    """``dy2 @ cat(owners)`` (input gradient of :func:`forward_product`) with both operands quantised."""
    w = owners[0] if len(owners) == 1 else lin_ops._fused_view(list(owners))
    return _dgrad(dy2, w, owners[0])


def usable(x2: torch.Tensor, owners: list[torch.Tensor]) -> bool:
    """FP8 execution applies: autocast active, weights marked, CUDA bf16, shapes fit the 128-wide scale blocks."""
    return (lin_ops.fp8_route(list(owners)) and kernel_ok(x2, *owners) and fp8_shapes_ok(list(owners))
            and sum(w.shape[0] for w in owners) % BLOCK == 0 and (len(owners) == 1 or lin_ops._adjacent(list(owners))))


class _Fp8Linear(torch.autograd.Function):
    """``y = x cat(W_i)^T + b``; the ``W_i`` are adjacent in memory (or a single matrix), so their
    concatenation is a view. Weight gradients go to each ``W_i`` (through ``main_grad`` when it has one)."""

    @staticmethod
    def forward(ctx, x, bias, *owners):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pre = getattr(x, "_fp8_rowwise", None)
        if pre is not None and x2 is not x:
            x2._fp8_rowwise = pre          # quantised by the producing norm launch
        w = owners[0] if len(owners) == 1 else lin_ops._fused_view(list(owners))
        T = x2.shape[0]
        # FP8 weight gradient: the transposed e4m3 copy of x (made in the same pass as the forward operand) is
        # what the backward keeps, instead of x itself
        ctx.fp8_wgrad = (fp8_wgrad_enabled() and T % BLOCK == 0 and x2.shape[1] % 16 == 0
                         and any(ctx.needs_input_grad[2:]))
        if ctx.fp8_wgrad:
            wq, ws, _ = _cached_weight_tensor(w, owners[0])
            xq, xs, xqt = _quantize_activation_t(x2, owners[0], "x")
            y = gemm_fp8_tensor(xq, xs, wq, ws)
            ctx.save_for_backward(xqt, xs, *owners)
        else:
            y = _fwd(x2, w, owners[0])
            ctx.save_for_backward(x2, *owners)
        if bias is not None:
            y = y + bias
        ctx.owners = owners
        ctx.has_bias = bias is not None
        ctx.x_shape = shp
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        owners = ctx.owners
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = db = None
        w = owners[0] if len(owners) == 1 else lin_ops._fused_view(list(owners))
        dws: list = [None] * len(owners)
        if ctx.fp8_wgrad:
            xqt, xs = ctx.saved_tensors[0], ctx.saved_tensors[1]
            dq, ds, dqt = _quantize_activation_t(dy2, owners[0], "dy")
            if ctx.needs_input_grad[0]:
                _, ws, wqt = _cached_weight_tensor(w, owners[0])
                dx = gemm_fp8_tensor(dq, ds, wqt, ws).view(ctx.x_shape)
            o = 0
            for i, p in enumerate(owners):
                rows = p.shape[0]
                if ctx.needs_input_grad[2 + i]:
                    mg = lin_ops.main_grad_of(p)
                    if mg is not None and mg.dtype == torch.bfloat16 and mg.stride(-1) == 1:
                        gemm_fp8_tensor(dqt[o:o + rows], ds, xqt, xs, out=mg, accumulate=lin_ops.main_grad_write(p))
                    elif mg is not None:
                        g = gemm_fp8_tensor(dqt[o:o + rows], ds, xqt, xs)
                        mg.add_(g) if lin_ops.main_grad_write(p) else mg.copy_(g)
                    else:
                        dws[i] = gemm_fp8_tensor(dqt[o:o + rows], ds, xqt, xs)
                o += rows
            if ctx.has_bias:
                db = dy2.float().sum(0).to(dy.dtype)
            return (dx, db, *dws)
        x2 = ctx.saved_tensors[0]
        if ctx.needs_input_grad[0]:
            dx = _dgrad(dy2, w, owners[0]).view(ctx.x_shape)
        o = 0
        for i, p in enumerate(owners):
            rows = p.shape[0]
            if ctx.needs_input_grad[2 + i]:
                mg = lin_ops.main_grad_of(p)
                if mg is not None:
                    gemm.gemm(dy2[:, o:o + rows], x2, a_mn=True, b_mn=True, out=mg, accumulate=lin_ops.main_grad_write(p))
                else:
                    dws[i] = gemm.gemm(dy2[:, o:o + rows], x2, a_mn=True, b_mn=True)
            o += rows
        if ctx.has_bias:
            db = dy2.float().sum(0).to(dy.dtype)
        return (dx, db, *dws)


def fp8_shapes_ok(weights: list[torch.Tensor]) -> bool:
    k = weights[0].shape[1]
    return k % BLOCK == 0 and sum(w.shape[0] for w in weights) % 16 == 0 and all(w.is_contiguous() for w in weights)


def fp8_linear(x: torch.Tensor, weights: torch.Tensor | list[torch.Tensor], bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ cat(weights)^T + bias`` through the block-scaled e4m3 GEMM. ``weights`` is one matrix or a
    list of matrices that sit back to back in memory. Falls back to the bf16 GEMM when shapes do not fit."""
    ws = [weights] if isinstance(weights, torch.Tensor) else list(weights)
    if kernel_ok(x, *ws) and fp8_shapes_ok(ws) and (len(ws) == 1 or lin_ops._adjacent(ws)):
        return _Fp8Linear.apply(x, bias, *ws)
    if len(ws) == 1:
        return lin_ops._MultiLinear.apply(x, 1, ws[0], bias) if lin_ops._kernel_ok(x, ws, [bias]) else \
            torch.nn.functional.linear(x, ws[0], bias)
    y = lin_ops._MultiLinear.apply(x, len(ws), *ws, *([None] * len(ws)))
    return y if bias is None else y + bias
