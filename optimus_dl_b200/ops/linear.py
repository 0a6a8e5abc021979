"""Linear layers on the tcgen05 GEMM, with opportunistic fusion of sibling projections.

``multi_linear(x, [Wq, Wk, Wv])`` returns ``x @ cat(W)^T``. When the weights are adjacent slices
of one flat buffer (which is how the sharding engine in ``parallel/fsdp.py`` lays a block out)
the concatenation is a free view and the three projections run as one GEMM; the weight gradient
is likewise one GEMM. Parameters keep their separate names and state-dict entries
(``attn.wq.weight`` ... as in optimus_dl/modules/model/blocks/attention.py:120-123).

Gradient placement: when a weight carries a ``main_grad`` tensor (a view into the engine's flat
gradient buffer) the weight-gradient GEMM writes (first micro-batch) or accumulates (later
micro-batches) straight into it and autograd receives no gradient for that weight, so no extra
copy or add pass over the gradients is needed.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gemm


def _adjacent(ts: list[torch.Tensor]) -> bool:
    """True when the 2-D row-major tensors are back-to-back in one storage with equal widths."""
    if len(ts) == 1:
        return ts[0].is_contiguous()
    k = ts[0].shape[1]
    for a, b in zip(ts[:-1], ts[1:]):
        if not (a.is_contiguous() and b.is_contiguous() and b.shape[1] == k and a.dtype == b.dtype):
            return False
        if a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
            return False
        if a.storage_offset() + a.numel() != b.storage_offset():
            return False
    return True


def _fused_view(ts: list[torch.Tensor]) -> torch.Tensor:
    rows = sum(t.shape[0] for t in ts)
    return ts[0].as_strided((rows, ts[0].shape[1]), (ts[0].shape[1], 1), ts[0].storage_offset())


def _adjacent_1d(ts: list[torch.Tensor]) -> bool:
    for a, b in zip(ts[:-1], ts[1:]):
        if a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr() or a.storage_offset() + a.numel() != b.storage_offset():
            return False
    return all(t.is_contiguous() for t in ts)


def main_grad_of(p: torch.Tensor) -> torch.Tensor | None:
    return getattr(p, "main_grad", None)


def main_grad_write(p: torch.Tensor) -> bool:
    """Returns whether the next write into ``p.main_grad`` must accumulate, and marks it written."""
    acc = bool(getattr(p, "_main_grad_filled", False))
    p._main_grad_filled = True
    return acc


class _MultiLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, n, *wb):
        ws = list(wb[:n])
        bs = list(wb[n:])
        has_bias = bs[0] is not None
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        sizes = [w.shape[0] for w in ws]
        job = getattr(ws[0], "_ag_pending", None)
        if job is not None and not job.done and _adjacent(ws):
            # the weight is still being gathered from its owners: the same launch pulls it over
            # NVLink and multiplies, tile by tile (parallel/fsdp.AGJob -> csrc/gemm_ag.cu)
            y = job.run(x2 if x2.is_contiguous() else x2.contiguous(), _fused_bias(bs) if has_bias else None)
        elif _adjacent(ws):
            wf = _fused_view(ws)
            bias = None
            if has_bias:
                bias = _fused_bias(bs)
            y = gemm.gemm(x2, wf, bias=bias)
        else:
            y = torch.empty((x2.shape[0], sum(sizes)), dtype=x.dtype, device=x.device)
            o = 0
            for w, b, s in zip(ws, bs, sizes):
                gemm.gemm(x2, w, bias=b, out=y[:, o:o + s])
                o += s
        ctx.save_for_backward(x2, *ws)
        ctx.n = n
        ctx.has_bias = has_bias
        ctx.sizes = sizes
        ctx.params = ws  # for main_grad lookup (attributes are not kept on saved tensors)
        ctx.x_shape = shp
        return y.view(*shp[:-1], sum(sizes))

    @staticmethod
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        x2, ws = saved[0], list(saved[1:])
        n, sizes = ctx.n, ctx.sizes
        params = ctx.params
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        fused = _adjacent(ws)
        if ctx.needs_input_grad[0]:
            if fused:
                dx = gemm.gemm(dy2, _fused_view(ws), b_mn=True)
            else:
                o = 0
                for i, (w, s) in enumerate(zip(ws, sizes)):
                    if i == 0:
                        dx = gemm.gemm(dy2[:, o:o + s], w, b_mn=True)
                    else:
                        gemm.gemm(dy2[:, o:o + s], w, b_mn=True, out=dx, accumulate=True)
                    o += s
            dx = dx.view(ctx.x_shape)
        dws: list = [None] * n
        mgs = [main_grad_of(p) for p in params]
        need = [ctx.needs_input_grad[2 + i] for i in range(n)]
        if any(need):
            if fused and all(m is not None for m in mgs) and _adjacent(mgs) and all(need):
                accs = [main_grad_write(p) for p in params]
                if all(accs) or not any(accs):
                    gemm.gemm(dy2, x2, a_mn=True, b_mn=True, out=_fused_view(mgs), accumulate=accs[0])
                else:  # mixed state: fall back to per-weight writes
                    o = 0
                    for p, m, s, a in zip(params, mgs, sizes, accs):
                        gemm.gemm(dy2[:, o:o + s], x2, a_mn=True, b_mn=True, out=m, accumulate=a)
                        o += s
            else:
                o = 0
                for i, (p, m, s) in enumerate(zip(params, mgs, sizes)):
                    if need[i]:
                        if m is not None:
                            gemm.gemm(dy2[:, o:o + s], x2, a_mn=True, b_mn=True, out=m, accumulate=main_grad_write(p))
                        else:
                            dws[i] = gemm.gemm(dy2[:, o:o + s], x2, a_mn=True, b_mn=True)
                    o += s
        dbs: list = [None] * n
        if ctx.has_bias:
            db = dy2.float().sum(0).to(dy.dtype)
            o = 0
            for i, s in enumerate(sizes):
                if ctx.needs_input_grad[2 + n + i]:
                    dbs[i] = db[o:o + s]
                o += s
        return (dx, None, *dws, *dbs)


def _fused_bias(bs: list[torch.Tensor]) -> torch.Tensor:
    if len(bs) == 1:
        return bs[0]
    if _adjacent_1d(bs):
        return bs[0].as_strided((sum(b.numel() for b in bs),), (1,), bs[0].storage_offset())
    return torch.cat(bs)


def _kernel_ok(x: torch.Tensor, ws: list[torch.Tensor], bs: list) -> bool:
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        return False
    if any(w.dtype != torch.bfloat16 or w.dim() != 2 or w.shape[1] % 8 != 0 for w in ws):
        return False
    if any(b is not None and b.dtype != torch.bfloat16 for b in bs):
        return False
    return sum(w.shape[0] for w in ws) % 8 == 0


def ensure_gathered(weights: list[torch.Tensor]) -> None:
    """Finish a pending fused all-gather of these weights when the consumer is not the fused AG GEMM."""
    job = getattr(weights[0], "_ag_pending", None)
    if job is not None and not job.done:
        job.gather_only()


def fp8_route(weights: list[torch.Tensor]) -> bool:
    """True when an FP8 autocast context is active and every weight was marked for FP8 execution
    (``_fp8`` attribute, set by the ``transformer_engine`` model transform)."""
    if not all(getattr(w, "_fp8", False) for w in weights):
        return False
    from ..amp.fp8 import fp8_enabled

    return fp8_enabled()


def _fp8_multi_linear(x: torch.Tensor, weights: list[torch.Tensor], biases: list) -> torch.Tensor:
    from . import fp8 as fp8_ops

    ensure_gathered(weights)
    if len(weights) == 1:
        return fp8_ops.fp8_linear(x, weights[0], biases[0])
    if _adjacent(weights):
        bias = None if biases[0] is None else _fused_bias(biases)
        return fp8_ops.fp8_linear(x, weights, bias)
    return torch.cat([fp8_ops.fp8_linear(x, w, b) for w, b in zip(weights, biases)], dim=-1)


def multi_linear(x: torch.Tensor, weights: list[torch.Tensor], biases: list | None = None) -> torch.Tensor:
    """``cat([x @ W_i^T + b_i], -1)`` with one GEMM when the weights are adjacent in memory."""
    n = len(weights)
    biases = list(biases) if biases is not None else [None] * n
    if all(b is None for b in biases):
        biases = [None] * n
    elif any(b is None for b in biases):
        raise ValueError("either every projection has a bias or none")
    if fp8_route(weights) and _kernel_ok(x, weights, biases):
        return _fp8_multi_linear(x, weights, biases)
    if _kernel_ok(x, weights, biases):
        return _MultiLinear.apply(x, n, *weights, *biases)
    return torch.cat([F.linear(x, w, b) for w, b in zip(weights, biases)], dim=-1)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight^T + bias`` (tcgen05 GEMM for CUDA bf16, ``F.linear`` otherwise)."""
    if fp8_route([weight]) and _kernel_ok(x, [weight], [bias]):
        return _fp8_multi_linear(x, [weight], [bias])
    if _kernel_ok(x, [weight], [bias]):
        return _MultiLinear.apply(x, 1, weight, bias)
    return F.linear(x, weight, bias)
