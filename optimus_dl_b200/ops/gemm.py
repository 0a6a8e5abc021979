"""bf16 GEMM on the tcgen05 tensor cores, and the autograd ``linear`` built on it.

``matmul_nt`` & friends call the persistent TMA + TMEM kernel in
``csrc/gemm_core.cuh``. A linear layer needs three products; all run on the same
kernel by choosing which operand is stored reduction-major:

* forward   ``y  = x  @ W^T``  : A = x  [M,K] K-major,  B = W  [N,K] K-major
* dgrad     ``dx = dy @ W``    : A = dy [M,N] K-major,  B = W  [N,K] read as MN-major
* wgrad     ``dW = dy^T @ x``  : A = dy [M,N] read as MN-major, B = x [M,K] read as MN-major

On CPU (tests, the fp32 oracle) the same functions fall back to ``torch.matmul``.
Replaces the cuBLAS calls behind ``nn.Linear`` in the reference
(optimus_dl/modules/model/blocks/attention.py:317-319,528; blocks/mlp.py:73-78).
"""

from __future__ import annotations

import torch

import os

from . import _lib

# Products with at least this many 256 x 256 tiles run on the two-SM kernel (csrc/gemm_2sm.cu): one tile per SM pair
# and wave. OB_GEMM_2SM=0 keeps everything on the one-SM kernel (kept for A/B measurements in ops/benchmark.py).
PAIR_MIN_TILES = 74
USE_2SM = os.environ.get("OB_GEMM_2SM", "1") != "0"

ACT = {"none": 0, "gelu": 1, "relu2": 2, "silu": 3}
SKINNY_M = 64   # inference-only products with at most this many rows are weight-streaming problems (see gemm())
# ... and go to csrc/gemm_skinny.cu when the weight has at least this many elements. Measured on B200 inside a CUDA-graph
# replay of a decode step: the kernel's fixed cost per launch (barrier set-up, TMEM allocation, first TMA round trip,
# cluster barrier of the split form) makes it 1.3x slower than the library on the 4 to 25 MB weights of a 1.7B model,
# and it reaches 0.83 of the library's time on the 622 MB vocabulary projection. Smaller weights use torch.matmul.
SKINNY_MIN_WEIGHT = int(os.environ.get("OB_SKINNY_MIN_WEIGHT", 16 * 1024 * 1024))


def _use_kernel(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts)


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    accumulate: bool = False,
    bias: torch.Tensor | None = None,
    act: str = "none",
    alpha: float = 1.0,
    b_flags: torch.Tensor | None = None,
    flag_rows: int = 0,
    flag_value: int = 0,
    a_flags: torch.Tensor | None = None,
    a_flag_rows: int = 0,
    a_flag_value: int = 0,
    tile_order: int = 0,
    first_tile_shift: int = 0,
    max_ctas: int = 0,
) -> torch.Tensor:
    """``C[M,N] = act(alpha * A B^T + bias)`` with bf16 inputs and fp32 accumulation.

    ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b`` is ``[N,K]`` (or ``[K,N]`` when
    ``b_mn``). ``out`` may be bf16 or fp32; with ``accumulate`` the product is added to it.
    """
    a = _row_major_2d(a)
    b = _row_major_2d(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an output tensor")
        if out_dtype is None:  # bf16 on the kernel path; the operand dtype for the eager fallback
            out_dtype = torch.bfloat16 if _use_kernel(a, b) else a.dtype
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError("bad output shape")
    if not _use_kernel(a, b) or out.dtype not in (torch.bfloat16, torch.float32):
        A = a.t() if a_mn else a
        Bt = b if b_mn else b.t()
        r = (A.float() @ Bt.float()) * alpha
        if bias is not None:
            r = r + bias.float()
        if act == "gelu":
            r = torch.nn.functional.gelu(r)
        elif act == "relu2":
            r = torch.relu(r) ** 2
        elif act == "silu":
            r = torch.nn.functional.silu(r)
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r.to(out.dtype))
        return out
    skinny = (M <= SKINNY_M and not a_mn and not accumulate and act == "none" and alpha == 1.0
              and out.dtype == torch.bfloat16 and b_flags is None and a_flags is None and not torch.is_grad_enabled())
    if skinny and (b_mn or N * K < SKINNY_MIN_WEIGHT) and out.is_contiguous():
        torch.matmul(a, b if b_mn else b.t(), out=out)
        if bias is not None:
            out.add_(bias)
        return out
    if skinny and not b_mn:
        # single-token decode steps: a handful of rows against a whole weight matrix is a weight-streaming
        # problem; csrc/gemm_skinny.cu puts 128 weight rows on the M side of the tensor-core product, the token
        # rows on its N side, and splits the reduction over the CTAs of a cluster when the weight has few row tiles
        l = _lib.lib()
        splits = int(l.ob_gemm_skinny_splits(N, K))
        rc = l.ob_gemm_skinny_bf16(_lib.ptr(a), a.stride(0), _lib.ptr(b), b.stride(0), _lib.ptr(out), out.stride(0),
                                   M, N, K, _lib.ptr(bias), splits,
                                   _lib.ptr(_lib.status_word(a.device)), _lib.stream())
        _lib.check(rc, "ob_gemm_skinny_bf16")
        return out
    l = _lib.lib()
    if (USE_2SM and b_flags is None and a_flags is None and tile_order == 0
            and ((M + 255) // 256) * ((N + 255) // 256) >= PAIR_MIN_TILES):
        rc = l.ob_gemm2_bf16(
            _lib.ptr(a), a.stride(0), int(a_mn), _lib.ptr(b), b.stride(0), int(b_mn),
            _lib.ptr(out), out.stride(0), M, N, K, int(out.dtype == torch.float32), int(accumulate),
            _lib.ptr(bias), ACT[act], float(alpha), int(max_ctas),
            _lib.ptr(_lib.status_word(a.device)), _lib.stream(),
        )
        _lib.check(rc, "ob_gemm2_bf16")
        return out
    rc = l.ob_gemm_bf16(
        _lib.ptr(a), a.stride(0), int(a_mn), _lib.ptr(b), b.stride(0), int(b_mn),
        _lib.ptr(out), out.stride(0), M, N, K, int(out.dtype == torch.float32), int(accumulate),
        _lib.ptr(bias), ACT[act], float(alpha),
        _lib.ptr(b_flags), int(flag_rows), int(flag_value),
        _lib.ptr(a_flags), int(a_flag_rows), int(a_flag_value),
        int(tile_order), int(first_tile_shift), int(max_ctas),
        _lib.ptr(_lib.status_word(a.device)), _lib.stream(),
    )
    _lib.check(rc, "ob_gemm_bf16")
    return out


def matmul_nt(x: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T``."""
    return gemm(x, w, **kw)


def matmul_nn(x: torch.Tensor, w: torch.Tensor, **kw) -> torch.Tensor:
    """``x[M,K] @ w[K,N]``."""
    return gemm(x, w, b_mn=True, **kw)


def matmul_tn(x: torch.Tensor, y: torch.Tensor, **kw) -> torch.Tensor:
    """``x[K,M]^T @ y[K,N]`` (the weight-gradient product)."""
    return gemm(x, y, a_mn=True, b_mn=True, **kw)


def swiglu_gemm(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, save_gu: bool = True):
    """``h = silu(x w1^T) * (x w2^T)`` in one kernel; returns ``(h, g, u)`` (g, u None unless saved)."""
    x2 = _row_major_2d(x)
    M, K = x2.shape
    N = w1.shape[0]
    if not _use_kernel(x2, w1, w2) or w1.stride(0) != w2.stride(0):
        g = (x2.float() @ w1.float().t()).to(x.dtype)
        u = (x2.float() @ w2.float().t()).to(x.dtype)
        h = (torch.nn.functional.silu(g.float()) * u.float()).to(x.dtype)
        return h, (g if save_gu else None), (u if save_gu else None)
    h = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    g = torch.empty_like(h) if save_gu else None
    u = torch.empty_like(h) if save_gu else None
    l = _lib.lib()
    fn = l.ob_gemm2_swiglu_bf16 if (USE_2SM and ((M + 255) // 256) * ((N + 127) // 128) >= PAIR_MIN_TILES) else l.ob_gemm_swiglu_bf16
    rc = fn(
        _lib.ptr(x2), x2.stride(0), _lib.ptr(w1), _lib.ptr(w2), w1.stride(0), _lib.ptr(h), _lib.ptr(g), _lib.ptr(u),
        h.stride(0), M, N, K, _lib.ptr(_lib.status_word(x.device)), _lib.stream(),
    )
    _lib.check(rc, "ob_gemm_swiglu_bf16")
    return h, g, u


def swiglu_bwd_gemm(dy: torch.Tensor, wc: torch.Tensor, g: torch.Tensor, u: torch.Tensor) -> bool:
    """``dh = dy @ wc`` fused with the SwiGLU backward: ``g <- dg``, ``u <- du`` in place, ``dh`` never stored.

    ``dy`` is ``[M, D]``, ``wc`` the down projection ``[D, F]``, ``g`` / ``u`` the saved ``[M, F]`` gate and up
    products. Returns False (and touches nothing) when the fused two-SM kernel does not apply; the caller then runs
    the GEMM and the elementwise kernel separately.

    The feed-forward block does NOT use this by default: at 8192 x 14336 x 4096 it measures 0.76 ms against 0.62 ms
    for the plain product plus 0.22 ms for the elementwise kernel, and the same step time in the 8B training step.
    The product runs at the L2 bandwidth its 256 x 256 tiles need (about 11 TB/s of operand reads), so the 0.9 GB
    that the epilogue reads and writes are not hidden under the main loop but add to it.
    """
    M, D = dy.shape
    F = wc.shape[1]
    ok = (
        USE_2SM
        and _use_kernel(dy, wc, g, u)
        and dy.is_contiguous() and g.is_contiguous() and u.is_contiguous() and wc.stride(1) == 1
        and g.shape == (M, F) and u.shape == (M, F) and wc.shape[0] == D
        and F % 8 == 0 and D % 8 == 0 and wc.stride(0) % 8 == 0
        and ((M + 255) // 256) * ((F + 255) // 256) >= PAIR_MIN_TILES
    )
    if not ok:
        return False
    rc = _lib.lib().ob_gemm2_swiglu_bwd_bf16(
        _lib.ptr(dy), dy.stride(0), _lib.ptr(wc), wc.stride(0), _lib.ptr(g), _lib.ptr(u), g.stride(0), M, F, D,
        _lib.ptr(_lib.status_word(dy.device)), _lib.stream(),
    )
    _lib.check(rc, "ob_gemm2_swiglu_bwd_bf16")
    return True


CE_STATS_MIN_K = int(os.environ.get("OB_CE_STATS_MIN_K", "4096"))


def ce_stats_gemm(x: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, stats: torch.Tensor, best_idx: torch.Tensor,
                  vocab_offset: int = 0, softcap_mode: int = 0, cap: float = 1.0) -> bool:
    """Per-row cross-entropy statistics of ``x @ w^T`` without the logits: the GEMM's epilogue reduces each 256-column
    tile to (max, sum-exp, sum, largest value and its column, target logit) and a small kernel folds the tiles.

    ``stats`` is a ``[5, rows]`` fp32 view filled as ``ob_ce_stats`` fills it (max, sum-exp, sum z, z[target], best
    value), ``best_idx`` the ``[rows]`` int32 arg-max (global column). Returns False, touching nothing, when the
    two-SM kernel does not apply; the caller then materialises the chunk's logits.

    Used for K >= ``CE_STATS_MIN_K`` only. The epilogue's 256 exponentials, comparisons and roundings per thread and
    tile take about 23 us on the four epilogue warps of a CTA; the main loop of a 256 x 256 tile hides that at
    K = 4096 (4096 x 128256 x 4096: 3.02 ms against 3.06 ms for the product plus the statistics kernel, with no 1 GB
    chunk of logits) but not at K = 2048 (4096 x 151936 x 2048: 3.00 ms against 2.40 ms).
    """
    rows, K = x.shape
    V = w.shape[0]
    ok = (
        USE_2SM and _use_kernel(x, w) and x.stride(1) == 1 and w.stride(1) == 1 and K % 8 == 0 and K >= CE_STATS_MIN_K
        and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and targets.dtype == torch.int64 and targets.is_contiguous()
        and ((rows + 255) // 256) * ((V + 255) // 256) >= PAIR_MIN_TILES
    )
    if not ok:
        return False
    l = _lib.lib()
    tiles_n = l.ob_gemm2_ce_tiles(V)
    part = torch.empty((rows, tiles_n, 4), dtype=torch.float32, device=x.device)
    part_idx = torch.empty((rows, tiles_n), dtype=torch.int32, device=x.device)
    stats[3].zero_()                      # rows whose target lies outside this vocabulary slice keep 0
    rc = l.ob_gemm2_ce_stats_bf16(
        _lib.ptr(x), x.stride(0), _lib.ptr(w), w.stride(0), rows, V, K, _lib.ptr(targets), _lib.ptr(part),
        _lib.ptr(part_idx), _lib.ptr(stats[3]), int(vocab_offset), int(softcap_mode), float(cap),
        _lib.ptr(_lib.status_word(x.device)), _lib.stream(),
    )
    _lib.check(rc, "ob_gemm2_ce_stats_bf16")
    rc = l.ob_ce_stats_merge(_lib.ptr(part), _lib.ptr(part_idx), rows, tiles_n, _lib.ptr(stats[0]), _lib.ptr(stats[1]),
                             _lib.ptr(stats[2]), _lib.ptr(stats[4]), _lib.ptr(best_idx), int(vocab_offset), _lib.stream())
    _lib.check(rc, "ob_ce_stats_merge")
    return True


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        shp = x.shape
        y = gemm(x.reshape(-1, shp[-1]), w, bias=bias)
        return y.view(*shp[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view_as(x)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Autograd-aware ``x @ w^T + bias``; tcgen05 kernel for CUDA bf16, ``F.linear`` otherwise."""
    if _use_kernel(x, w) and (bias is None or bias.dtype == torch.bfloat16):
        return _Linear.apply(x, w, bias)
    return torch.nn.functional.linear(x, w, bias)
