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


def bench_attention(t: Timer, cases) -> None:
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True, choices=["gemm_bf16", "gemm_skinny", "gemm_fp8", "attention", "decode", "sampler", "elementwise",
                                                    "tp_ag_gemm", "tp_gemm_rs", "tp_ag_gemm_fp8", "tp_gemm_rs_fp8"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true", help="one small case (for profiler captures)")
    ap.add_argument("--mid", action="store_true", help="attention: one case that fills every SM but holds little memory "
                                                        "(T 4096, 32 / 8 heads), for profiler captures")
    args = ap.parse_args()
    t = Timer(args.iters)
    if args.op == "gemm_bf16":
        bench_gemm_bf16(t, [(4096, 4096, 4096)] if args.small else [(8192, 8192, 8192), (8192, 6144, 4096), (8192, 4096, 14336),
                                                                    (8192, 28672, 4096)])
    elif args.op == "gemm_skinny":   # decode-step shapes of a 1.7B model at batch 64: weight-streaming bound
        bench_gemm_bf16(t, [(64, 4096, 2048), (64, 12288, 2048), (64, 2048, 6144), (64, 151936, 2048), (8, 4096, 4096)])
    elif args.op == "gemm_fp8":
        bench_gemm_fp8(t, [(4096, 4096, 4096)] if args.small else [(8192, 8192, 8192), (8192, 6144, 4096), (8192, 4096, 14336),
                                                                   (8192, 28672, 4096)])
    elif args.op == "attention":
        bench_attention(t, [(4096, 32, 8, 128)] if args.mid else [(4096, 8, 2, 128)] if args.small
                        else [(8192, 32, 8, 128), (16384, 40, 8, 128)])
    elif args.op == "decode":
        bench_decode(t, [(64, 768, 16, 8, 128)] if args.small else [(64, 768, 16, 8, 128), (512, 768, 16, 8, 128),
                                                                     (1, 8192, 32, 8, 128), (8, 4096, 32, 8, 128)])
    elif args.op == "elementwise":
        bench_elementwise(t)
    elif args.op == "sampler":
        bench_sampler(t, [(64, 151936)] if args.small else [(64, 151936), (512, 151936)])
    else:
        bench_tp(args.op, t, [(8192, 6144, 4096), (16384, 5120, 17408 // 2), (16384, 17408 // 2, 5120)])


if __name__ == "__main__":
    main()
