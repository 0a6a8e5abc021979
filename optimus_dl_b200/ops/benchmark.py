"""Kernel micro-benchmarks: ``python -m optimus_dl_b200.ops.benchmark --op <name> [--size ...]``.

Every case is timed with CUDA events on the launching stream after warm-up, with a synchronise on
both sides; between timed iterations a buffer larger than the L2 cache is overwritten, so no case
reads its operands from a warm L2. One JSON line per case: the achieved rate, the algorithmic work
it is computed from, and (when ``MEASURED_PEAKS.json`` is found next to the repository root) the
fraction of the measured copy bandwidth / cuBLAS bf16 throughput. Multi-GPU cases
(``--op tp_ag_gemm`` / ``tp_gemm_rs``) are launched with ``torchrun`` and report the maximum over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
from typing import Callable

import torch


def _peaks() -> dict:
    here = os.path.dirname(os.path.abspath(__file__))
    for up in (3, 2):
        p = os.path.join(here, *[".."] * (up - 1), "MEASURED_PEAKS.json")
        if os.path.exists(p):
            try:
                return json.load(open(p))
            except Exception:  # noqa: BLE001
                return {}
    return {}


class Timer:
    def __init__(self, iters: int = 20, warmup: int = 3, flush_mb: int = 512):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(flush_mb * 1024 * 1024 // 4, dtype=torch.float32, device="cuda") if flush_mb else None

    def __call__(self, fn: Callable[[], None]) -> float:
        """Median milliseconds per call."""
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.add_(1.0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        times.sort()
        return times[len(times) // 2]


def _emit(op: str, case: dict, ms: float, flops: float = 0.0, bytes_: float = 0.0, **extra) -> None:
    pk = _peaks()
    rec = {"op": op, **case, "ms": round(ms, 4)}
    if flops:
        tf = flops / ms / 1e9
        rec["tflops"] = round(tf, 1)
        if pk.get("bf16_tflops"):
            rec["of_measured_bf16_peak"] = round(tf / pk["bf16_tflops"], 3)
    if bytes_:
        gbs = bytes_ / ms / 1e6
        rec["gbs"] = round(gbs, 1)
        if pk.get("hbm_gbs"):
            rec["of_measured_hbm"] = round(gbs / pk["hbm_gbs"], 3)
    rec.update(extra)
    print(json.dumps(rec), flush=True)


def bench_gemm_bf16(t: Timer, sizes) -> None:
    """Forward layout (A and B reduction-major) for every size, then the dgrad (B read MN-major) and wgrad (both
    operands MN-major, K = tokens) layouts of the flagship MLP shapes; each against ``torch.matmul`` on the same
    operands, and with the one-SM kernel for comparison where the two-SM kernel is the default."""
    from . import gemm

    def run(tag, M, N, K, a, b, a_mn, b_mn, ref):
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: gemm.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out))
        saved, gemm.USE_2SM = gemm.USE_2SM, False
        ms1 = t(lambda: gemm.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out))
        gemm.USE_2SM = saved
        ms_ref = t(lambda: ref(out))
        _emit("gemm_bf16", dict(layout=tag, M=M, N=N, K=K), ms, flops=2.0 * M * N * K, one_sm_kernel_ms=round(ms1, 4),
              cublas_ms=round(ms_ref, 4), vs_cublas=round(ms_ref / ms, 3))

    for M, N, K in sizes:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        run("fwd  x[M,K] w[N,K]^T", M, N, K, a, b, False, False, lambda o: torch.matmul(a, b.t(), out=o))
    if len(sizes) > 1:
        for M, N, K in [(8192, 14336, 4096), (8192, 4096, 14336)]:
            a = torch.randn(M, K, device="cuda").bfloat16()
            w = torch.randn(K, N, device="cuda").bfloat16()      # dgrad: dy[M,K] @ W[K,N], W read MN-major
            run("dgrad dy[M,K] w[K,N]", M, N, K, a, w, False, True, lambda o: torch.matmul(a, w, out=o))
        for M, N, K in [(14336, 4096, 8192), (4096, 14336, 8192), (6144, 4096, 8192)]:
            dy = torch.randn(K, M, device="cuda").bfloat16()     # wgrad: dy[K,M]^T @ x[K,N]
            x = torch.randn(K, N, device="cuda").bfloat16()
            run("wgrad dy[K,M]^T x[K,N]", M, N, K, dy, x, True, True, lambda o: torch.matmul(dy.t(), x, out=o))
        M, N, K = 8192, 14336, 4096
        x = torch.randn(M, K, device="cuda").bfloat16()
        w1 = torch.randn(N, K, device="cuda").bfloat16()
        w2 = torch.randn(N, K, device="cuda").bfloat16()
        ms = t(lambda: gemm.swiglu_gemm(x, w1, w2))
        saved, gemm.USE_2SM = gemm.USE_2SM, False
        ms1 = t(lambda: gemm.swiglu_gemm(x, w1, w2))
        gemm.USE_2SM = saved
        g = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        u = torch.empty_like(g)

        def lib():
            torch.matmul(x, w1.t(), out=g)
            torch.matmul(x, w2.t(), out=u)
            return torch.nn.functional.silu(g) * u

        _emit("gemm_swiglu_dual_b", dict(M=M, N=N, K=K), ms, flops=4.0 * M * N * K, one_sm_kernel_ms=round(ms1, 4),
              cublas_plus_eager_ms=round(t(lib), 4))


def bench_gemm_skinny(t: Timer, sizes) -> None:
    """Decode-step products (M <= 64 rows): the weight-streaming kernel against ``torch.matmul``; the rate is the
    weight bytes over the time, to be read against the measured copy bandwidth."""
    from . import gemm

    gemm.SKINNY_MIN_WEIGHT = 0      # measure the kernel at every size (gemm() sends small weights to the library)
    for M, N, K in sizes:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        with torch.no_grad():
            ms = t(lambda: gemm.gemm(a, b, out=out))
            ms_ref = t(lambda: torch.matmul(a, b.t(), out=out))
        _emit("gemm_skinny", dict(M=M, N=N, K=K), ms, bytes_=2.0 * N * K + 2.0 * M * (N + K), cublas_ms=round(ms_ref, 4),
              vs_cublas=round(ms_ref / ms, 3))


def bench_gemm_fp8(t: Timer, sizes) -> None:
    from . import fp8

    for M, N, K in sizes:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
        a8, sa = fp8.quantize_rowwise(a)
        b8, sb = fp8.quantize_block(b)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = t(lambda: fp8.gemm_fp8(a8, sa, b8, sb, out=out))
        msq = t(lambda: fp8.quantize_rowwise(a))
        _emit("gemm_fp8_block", dict(M=M, N=N, K=K), ms, flops=2.0 * M * N * K, quant_rowwise_ms=round(msq, 4),
              quant_gbs=round(M * K * 3 / msq / 1e6, 1))
        t8, st = fp8.quantize_tensor(a)
        w8, sw, _ = fp8.quantize_weight_tensor(b)
        ms = t(lambda: fp8.gemm_fp8_tensor(t8, st, w8, sw, out=out))
        ms_cur = t(lambda: fp8.quantize_tensor(a))
        ms_del = t(lambda: fp8.quantize_tensor(a, scale=st))
        ms_t = t(lambda: fp8.quantize_tensor_t(a, scale=st))
        _emit("gemm_fp8_tensor", dict(M=M, N=N, K=K), ms, flops=2.0 * M * N * K, quant_current_ms=round(ms_cur, 4),
              quant_given_scale_ms=round(ms_del, 4), quant_given_scale_gbs=round(M * K * 3 / ms_del / 1e6, 1),
              quant_with_transpose_ms=round(ms_t, 4), quant_with_transpose_gbs=round(M * K * 4 / ms_t / 1e6, 1))


def bench_gemm_swiglu_bwd(t: Timer, T: int, D: int, F: int) -> None:
    """dh = dy Wc followed by the SwiGLU backward: the plain product, product + elementwise kernel, and the fused form."""
    from . import _lib, gemm

    dy = (torch.randn(T, D, device="cuda") * 0.5).bfloat16()
    wc = (torch.randn(D, F, device="cuda") * 0.05).bfloat16()
    g = torch.randn(T, F, device="cuda").bfloat16()
    u = torch.randn(T, F, device="cuda").bfloat16()
    h = torch.empty_like(g)

    def two_kernels():
        dh = gemm.gemm(dy, wc, b_mn=True)
        _lib.check(_lib.lib().ob_swiglu_bwd(_lib.ptr(dh), _lib.ptr(g), _lib.ptr(u), _lib.ptr(g), _lib.ptr(u), _lib.ptr(h),
                                            g.numel(), _lib.stream()), "swiglu_bwd")

    ms_plain = t(lambda: gemm.gemm(dy, wc, b_mn=True))
    ms_two = t(two_kernels)
    ms_fused = t(lambda: gemm.swiglu_bwd_gemm(dy, wc, g, u))
    _emit("gemm_swiglu_bwd", dict(M=T, N=F, K=D), ms_fused, flops=2.0 * T * F * D, plain_product_ms=round(ms_plain, 4),
          product_plus_elementwise_ms=round(ms_two, 4))
    _lib.check_status()


def bench_linear_ce_stats(t: Timer, cases) -> None:
    """Cross-entropy statistics of one row chunk of the head without gradients: logits written by the GEMM and read by
    the statistics kernel, against the GEMM whose epilogue reduces its tiles to the statistics."""
    from . import _lib, gemm

    gemm.CE_STATS_MIN_K = 0          # measure the fused form at every K (the dispatch keeps small K on two kernels)
    for rows, d, V in cases:
        x = (torch.randn(rows, d, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(V, d, device="cuda") * 0.05).bfloat16()
        tg = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int64)
        st = torch.empty(5, rows, device="cuda", dtype=torch.float32)
        bi = torch.empty(rows, device="cuda", dtype=torch.int32)
        ld = (V + 7) // 8 * 8
        buf = torch.empty(rows, ld, device="cuda", dtype=torch.bfloat16)
        out_view = buf.as_strided((rows, V), (ld, 1))
        l = _lib.lib()

        def two_kernels():
            gemm.gemm(x, w, out=out_view)
            _lib.check(l.ob_ce_stats(_lib.ptr(out_view), ld, _lib.ptr(tg), _lib.ptr(st[0]), _lib.ptr(st[1]), _lib.ptr(st[2]),
                                     _lib.ptr(st[3]), _lib.ptr(st[4]), _lib.ptr(bi), rows, V, 0, 0, 1.0, _lib.stream()), "ce_stats")

        ms_two = t(two_kernels)
        ms_fused = t(lambda: gemm.ce_stats_gemm(x, w, tg, st, bi))
        _emit("linear_ce_stats", dict(rows=rows, d=d, V=V), ms_fused, flops=2.0 * rows * d * V,
              gemm_plus_stats_kernel_ms=round(ms_two, 4))
        _lib.check_status()


def bench_attention(t: Timer, cases, library_rows: bool = True) -> None:
    from . import attention as A

    for T, Hq, Hk, hd in cases:
        qkv = torch.randn(1, T, (Hq + 2 * Hk) * hd, device="cuda").bfloat16().requires_grad_(True)
        ds = A.build_doc_start(1, T, qkv.device, None, None)
        flops_f = 4.0 * T * T * Hq * hd / 2   # causal: half of the score matrix
        out = A.qkv_attention(qkv, n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=ds)
        dout = torch.randn_like(out)
        ms_f = t(lambda: A.qkv_attention(qkv.detach(), n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=ds))
        _emit("attention_fwd", dict(T=T, Hq=Hq, Hk=Hk, hd=hd), ms_f, flops=flops_f)

        def fb():
            qkv.grad = None
            o = A.qkv_attention(qkv, n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=ds)
            o.backward(dout)

        ms_fb = t(fb)
        _emit("attention_fwd_bwd", dict(T=T, Hq=Hq, Hk=Hk, hd=hd), ms_fb, flops=flops_f * 3.5)
        if not library_rows:
            continue
        # the kernels the reference reaches for the same problem (optimus_dl/modules/model/blocks/attention.py:
        # flash_attn_varlen_func at 390-401, scaled_dot_product_attention at 511-520), same harness
        q = torch.randn(1, T, Hq, hd, device="cuda").bfloat16().requires_grad_(True)
        k = torch.randn(1, T, Hk, hd, device="cuda").bfloat16().requires_grad_(True)
        v = torch.randn(1, T, Hk, hd, device="cuda").bfloat16().requires_grad_(True)
        do = torch.randn(1, T, Hq, hd, device="cuda").bfloat16()
        libs = {}
        try:
            from flash_attn import flash_attn_func

            libs["flash_attn"] = lambda: flash_attn_func(q, k, v, causal=True)
        except Exception:  # noqa: BLE001
            pass
        qt, kt, vt = (x.transpose(1, 2) for x in (q, k, v))
        libs["torch_sdpa"] = lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True)
        for name, fwd in libs.items():
            try:
                with torch.no_grad():
                    ms_lf = t(fwd)

                def lfb():
                    q.grad = k.grad = v.grad = None
                    o = fwd()
                    o.backward(do if o.shape == do.shape else do.transpose(1, 2))

                ms_lfb = t(lfb)
                _emit(f"attention_library_{name}", dict(T=T, Hq=Hq, Hk=Hk, hd=hd), ms_lfb, flops=flops_f * 3.5,
                      fwd_ms=round(ms_lf, 4), fwd_tflops=round(flops_f / ms_lf / 1e9, 1))
            except Exception as e:  # noqa: BLE001
                print(json.dumps({"op": f"attention_library_{name}", "error": str(e)[:200]}), flush=True)


def bench_decode(t: Timer, cases) -> None:
    from . import decode as D

    for B, T, Hq, Hk, hd in cases:
        kc = torch.randn(B, Hk, T, hd, device="cuda").bfloat16().permute(0, 2, 1, 3)   # head-major storage
        vc = torch.randn(B, Hk, T, hd, device="cuda").bfloat16().permute(0, 2, 1, 3)
        qkv = torch.randn(B, (Hq + 2 * Hk) * hd, device="cuda").bfloat16()
        q = qkv[:, : Hq * hd].unflatten(1, (Hq, hd))
        kn = qkv[:, Hq * hd:(Hq + Hk) * hd].unflatten(1, (Hk, hd))
        vn = qkv[:, (Hq + Hk) * hd:].unflatten(1, (Hk, hd))
        lens = torch.full((B,), T, dtype=torch.int32, device="cuda")
        ctas = B * Hk
        splits = max(1, min(32, (12 * 148 + ctas - 1) // ctas, (T + 127) // 128))
        ws: dict = {}
        ms = t(lambda: D.decode_attention(q, kn, vn, kc, vc, lens, n_splits=splits, workspace=ws))
        _emit("decode_attention", dict(B=B, T=T, Hq=Hq, Hk=Hk, hd=hd, splits=splits), ms, bytes_=2.0 * B * T * Hk * hd * 2)


def bench_sampler(t: Timer, cases) -> None:
    from . import decode as D

    for B, V in cases:
        logits = torch.randn(B, V, device="cuda")
        for kw in (dict(), dict(top_k=50), dict(top_p=0.9)):
            ms = t(lambda: D.sample(logits, temperature=1.0, seed=1, offset=0, **kw))
            ms_ref = t(lambda: D.sample_ref(logits, 1.0, kw.get("top_k"), kw.get("top_p")))
            _emit("sampler", dict(B=B, V=V, **kw), ms, bytes_=4.0 * B * V, torch_ms=round(ms_ref, 4))


def bench_elementwise(t: Timer) -> None:
    from . import activation as act
    from . import norm

    M, F, D = 8192, 14336, 4096
    g = torch.randn(M, F, device="cuda").bfloat16()
    u = torch.randn(M, F, device="cuda").bfloat16()
    dh = torch.randn(M, F, device="cuda").bfloat16()
    ms = t(lambda: act.swiglu_backward(dh, g, u))
    _emit("swiglu_bwd", dict(rows=M, cols=F), ms, bytes_=5.0 * M * F * 2)
    x = torch.randn(M, D, device="cuda").bfloat16().requires_grad_(True)
    w = torch.ones(D, device="cuda").bfloat16().requires_grad_(True)
    ms = t(lambda: norm.rms_norm(x.detach(), w.detach(), 1e-5))
    _emit("rmsnorm_fwd", dict(rows=M, D=D), ms, bytes_=2.0 * M * D * 2)
    y = norm.rms_norm(x, w, 1e-5)
    dy = torch.randn_like(y)

    def bwd():
        x.grad = None
        w.grad = None
        y.backward(dy, retain_graph=True)

    ms = t(bwd)
    _emit("rmsnorm_bwd", dict(rows=M, D=D), ms, bytes_=3.0 * M * D * 2)


def bench_tp(op: str, t: Timer, cases) -> None:
    """All-gather + GEMM and GEMM + reduce-scatter against NCCL collective followed by / following the plain GEMM."""
    import torch.distributed as dist

    from ..parallel import tp as T
    from . import gemm

    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl")
    world = dist.get_world_size()
    state = T.TPState(dist.group.WORLD, torch.device("cuda", rank), sequence_parallel=True)
    for M, N, K in cases:
        rows = M // world
        if op == "tp_ag_gemm":
            x = torch.randn(rows, K, device="cuda").bfloat16()
            w = torch.randn(N, K, device="cuda").bfloat16()
            fused = lambda: T.ag_gemm(state, x, w, site=("bench", M, N, K))  # noqa: E731

            def base():
                xf = T.all_gather_rows(state, x)
                return gemm.gemm(xf, w)
        elif op == "tp_ag_gemm_fp8":
            from . import fp8

            x = torch.randn(rows, K, device="cuda").bfloat16()
            w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
            fused = lambda: T.ag_gemm_fp8(state, x, [w], ("bench", M, N, K))  # noqa: E731

            def base():   # bf16 all-gather, quantiser launch, FP8 GEMM
                xf = T.all_gather_rows(state, x)
                return fp8.forward_product(xf, [w])
        elif op == "tp_gemm_rs_fp8":
            from . import fp8

            x = torch.randn(M, K, device="cuda").bfloat16()
            w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
            fused = lambda: T.gemm_rs_fp8(state, x, [w])  # noqa: E731

            def base():
                return T.reduce_scatter_rows(state, fp8.forward_product(x, [w]))
        else:
            x = torch.randn(M, K, device="cuda").bfloat16()
            w = torch.randn(N, K, device="cuda").bfloat16()
            fused = lambda: T.gemm_rs(state, x, w)  # noqa: E731

            def base():
                return T.reduce_scatter_rows(state, gemm.gemm(x, w))

        x_plain = x if op in ("tp_gemm_rs", "tp_gemm_rs_fp8") else torch.randn(M, K, device="cuda").bfloat16()

        def stream_time(fn, reps: int = 10) -> float:
            """Per-call milliseconds of ``reps`` calls issued back to back: ranks stay in lockstep through the
            collectives themselves, so host-side launch skew between the processes is not part of the number.
            Operands and outputs of consecutive calls (> 126 MB together) do not fit in L2."""
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        if op in ("tp_ag_gemm_fp8", "tp_gemm_rs_fp8"):
            a8, sa = fp8.quantize_rowwise(x_plain)
            w8, sw, _, _ = fp8._cached_weight(w)
            ms_plain = stream_time(lambda: fp8.gemm_fp8(a8, sa, w8, sw))
        else:
            ms_plain = stream_time(lambda: gemm.gemm(x_plain, w))
        vals = torch.tensor([stream_time(fused), stream_time(base), ms_plain], device="cuda")
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        if dist.get_rank() == 0:
            link_bytes = (world - 1) / world * M * (N * 2 if op in ("tp_gemm_rs", "tp_gemm_rs_fp8") else K * (1 if op == "tp_ag_gemm_fp8" else 2))
            roof_ms = max(2.0 * M * N * K / (_peaks().get("bf16_tflops", 1590.0) * 1e9), link_bytes / 770e6)
            _emit(op, dict(M=M, N=N, K=K, world=world), float(vals[0]), flops=2.0 * M * N * K,
                  nccl_then_gemm_ms=round(float(vals[1]), 4), gemm_only_ms=round(float(vals[2]), 4),
                  roofline_ms=round(roof_ms, 4), of_roofline=round(roof_ms / float(vals[0]), 3))
    torch.cuda.synchronize()
    _ = state
    dist.barrier()
    dist.destroy_process_group()


def bench_fsdp(op: str, cases) -> None:
    """The two fused kernels of the fully-sharded engine on one Llama-3-8B-sized transformer block, against the
    library sequence they replace (launch with torchrun; maximum over ranks):

    * ``fsdp_ag_gemm``: the rows of the fused QKV weight are pulled from their owners by copy CTAs inside the QKV GEMM
      launch (``ob_gemm_ag_bf16``) vs NCCL all-gather of the weight followed by this package's GEMM;
    * ``fsdp_rs_adamw``: cross-GPU barrier + reduce-scatter of the block's bf16 gradients in fp32 + AdamW on the fp32
      shard + bf16 parameter refresh in one kernel (``ob_rs_adamw``) vs NCCL reduce-scatter + the stand-alone fused
      AdamW kernel (``ob_adamw``).

    Roofline = the slower of (FLOPs at the measured GEMM peak | HBM bytes at the measured copy bandwidth) and the
    bytes that must cross NVLink into this GPU at 770 GB/s."""
    import torch.distributed as dist
    import torch.nn as nn

    from ..parallel import fsdp
    from . import gemm
    from . import optim as optim_ops

    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    pk = _peaks()
    peak_tf, peak_bw, link = pk.get("bf16_tflops", 1590.0), pk.get("hbm_gbs", 6650.0), 770.0

    class Attn(nn.Module):
        def __init__(self, d, hq, hk, hd):
            super().__init__()
            self.wq = nn.Linear(d, hq * hd, bias=False)
            self.wk = nn.Linear(d, hk * hd, bias=False)
            self.wv = nn.Linear(d, hk * hd, bias=False)
            self.wo = nn.Linear(hq * hd, d, bias=False)

    class Block(nn.Module):
        def __init__(self, d, hq, hk, hd, f):
            super().__init__()
            self.attn = Attn(d, hq, hk, hd)
            self.w1 = nn.Linear(d, f, bias=False)
            self.w2 = nn.Linear(d, f, bias=False)
            self.c_proj = nn.Linear(f, d, bias=False)
            self.ln_1 = nn.Parameter(torch.ones(d))
            self.ln_2 = nn.Parameter(torch.ones(d))

    class Net(nn.Module):
        def __init__(self, *a):
            super().__init__()
            self.h = nn.ModuleList([Block(*a)])

        def fully_shard(self, **_):
            return list(self.h)

    def stream_time(fn, reps: int = 10) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    for T, d, hq, hk, hd, f in cases:
        torch.manual_seed(0)
        with torch.device(dev):
            net = Net(d, hq, hk, hd, f).to(torch.bfloat16)
        eng = fsdp.fully_shard_model(net, dist.group.WORLD if world > 1 else None, dev, fsdp.FSDPConfig())
        g = eng.groups[0]
        P = sum(i.param.numel() for i in g.infos)
        if op == "fsdp_ag_gemm":
            x = torch.randn(T, d, device=dev).bfloat16()
            nq = (hq + 2 * hk) * hd

            def fused():
                g.invalidate()
                g.slot.owner = g
                g.epoch += 1
                job = fsdp.AGJob(g, eng.cfg.copy_ctas)
                return job.run(x, None) if world > 1 else gemm.gemm(x, g.fused_weight())

            shard_rows = torch.randn(nq // world, d, device=dev).bfloat16()
            full = torch.empty(nq, d, device=dev, dtype=torch.bfloat16)

            def base():
                if world > 1:
                    dist.all_gather_into_tensor(full, shard_rows)
                return gemm.gemm(x, full)

            ms_gemm = stream_time(lambda: gemm.gemm(x, full))
            vals = torch.tensor([stream_time(fused), stream_time(base), ms_gemm], device=dev)
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
            flops = 2.0 * T * nq * d
            link_bytes = (world - 1) / world * nq * d * 2
            roof = max(flops / (peak_tf * 1e9), link_bytes / (link * 1e6))
            if dist.get_rank() == 0:
                _emit(op, dict(tokens=T, qkv_rows=nq, d_model=d, world=world), float(vals[0]), flops=flops,
                      nccl_all_gather_then_gemm_ms=round(float(vals[1]), 4), gemm_only_ms=round(float(vals[2]), 4),
                      roofline_ms=round(roof, 4), of_roofline=round(roof / float(vals[0]), 3))
        else:
            g.ensure_state()
            hp = dict(lr=1e-4, betas=(0.9, 0.95), eps=1e-8)
            g.grad_slot.tensor.normal_(0, 1e-3)
            state = {"n": 0}

            def fused():
                state["n"] += 1
                eng.barrier()
                g.rs_adamw(0, hp, state["n"], 1.0 / world)

            shard_g = torch.empty(g.flat_numel // world, device=dev, dtype=torch.bfloat16)
            gfull = g.grad_slot.tensor[: g.flat_numel // world * world]
            m = torch.zeros(shard_g.numel(), device=dev)
            v = torch.zeros_like(m)
            w32 = torch.zeros_like(m)
            wlp = torch.empty_like(shard_g)

            def base():
                state["n"] += 1
                if world > 1:
                    dist.reduce_scatter_tensor(shard_g, gfull)
                src = shard_g if world > 1 else gfull
                optim_ops.adamw_step_(w32, m, v, src, wlp, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0,
                                      step=state["n"], grad_scale=1.0 / world)

            vals = torch.tensor([stream_time(fused), stream_time(base)], device=dev)
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
            shard = P / world
            hbm_bytes = shard * 28.0 + (world - 1) / world * P * 2.0      # own shard state + serving the peers' reads
            link_bytes = (world - 1) * shard * 2.0                        # this rank's rows pulled from every peer
            roof = max(hbm_bytes / (peak_bw * 1e6), link_bytes / (link * 1e6))
            if dist.get_rank() == 0:
                _emit(op, dict(block_params=P, world=world), float(vals[0]), bytes_=hbm_bytes,
                      nccl_reduce_scatter_then_adamw_ms=round(float(vals[1]), 4), nvlink_bytes_in=int(link_bytes),
                      roofline_ms=round(roof, 4), of_roofline=round(roof / float(vals[0]), 3))
        _lib_check(dev)
        del eng, net
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def _lib_check(dev) -> None:
    from . import _lib

    _lib.check_status(dev)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm_bf16", "gemm_skinny", "gemm_swiglu_bwd", "linear_ce_stats", "gemm_fp8", "attention", "decode", "sampler", "elementwise",
                                                    "tp_ag_gemm", "tp_gemm_rs", "tp_ag_gemm_fp8", "tp_gemm_rs_fp8",
                                                    "fsdp_ag_gemm", "fsdp_rs_adamw"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true", help="one small case (for profiler captures)")
    ap.add_argument("--mid", action="store_true", help="attention: one case that fills every SM but holds little memory "
                                                        "(T 4096, 32 / 8 heads), for profiler captures")
    ap.add_argument("--no-library-rows", action="store_true", help="attention: skip the flash-attn / SDPA comparison rows "
                                                                    "(profiler captures of this package's kernels only)")
    args = ap.parse_args()
    if "LOCAL_RANK" in os.environ:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    t = Timer(args.iters)
    if args.op == "gemm_bf16":
        bench_gemm_bf16(t, [(4096, 4096, 4096)] if args.small else [(8192, 8192, 8192), (8192, 6144, 4096), (8192, 4096, 14336),
                                                                    (8192, 28672, 4096)])
    elif args.op == "gemm_swiglu_bwd":
        bench_gemm_swiglu_bwd(t, 8192, 4096, 14336)
    elif args.op == "linear_ce_stats":      # one 4096-row chunk of the output head: Llama-3-8B and Qwen3-1.7B
        bench_linear_ce_stats(t, [(4096, 4096, 128256), (4096, 2048, 151936)])
    elif args.op == "gemm_skinny":   # decode-step shapes of a 1.7B model at batch 64: weight-streaming bound
        bench_gemm_skinny(t, [(64, 4096, 2048), (64, 12288, 2048), (64, 2048, 6144), (64, 151936, 2048), (8, 4096, 4096)])
    elif args.op == "gemm_fp8":
        bench_gemm_fp8(t, [(4096, 4096, 4096)] if args.small else [(8192, 8192, 8192), (8192, 6144, 4096), (8192, 4096, 14336),
                                                                   (8192, 28672, 4096)])
    elif args.op == "attention":
        bench_attention(t, [(4096, 32, 8, 128)] if args.mid else [(4096, 8, 2, 128)] if args.small
                        else [(8192, 32, 8, 128), (16384, 40, 8, 128)], library_rows=not args.no_library_rows)
    elif args.op == "decode":
        bench_decode(t, [(64, 768, 16, 8, 128)] if args.small else [(64, 768, 16, 8, 128), (512, 768, 16, 8, 128),
                                                                     (1, 8192, 32, 8, 128), (8, 4096, 32, 8, 128)])
    elif args.op == "elementwise":
        bench_elementwise(t)
    elif args.op == "sampler":
        bench_sampler(t, [(64, 151936)] if args.small else [(64, 151936), (512, 151936)])
    elif args.op in ("fsdp_ag_gemm", "fsdp_rs_adamw"):
        # one Llama-3-8B block: 8192 tokens, d_model 4096, 32 / 8 heads of 128, FFN 14336
        bench_fsdp(args.op, [(8192, 4096, 32, 8, 128, 14336)])
    else:
        bench_tp(args.op, t, [(8192, 6144, 4096), (16384, 5120, 17408 // 2), (16384, 17408 // 2, 5120)])


if __name__ == "__main__":
    main()
