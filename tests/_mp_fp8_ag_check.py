"""Worker: fused quantise + e4m3 all-gather + GEMM against all-gather, quantiser launch and FP8 GEMM.
Run under torchrun-style environment variables as ``python _mp_fp8_ag_check.py <port>``."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = sys.argv[1]
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    dev = torch.device("cuda", rank)

    from optimus_dl_b200.amp.fp8 import FP8Recipe, Fp8Format, parse_fp8_recipe
    from optimus_dl_b200.ops import _lib, fp8
    from optimus_dl_b200.parallel import tp as T

    state = T.TPState(dist.group.WORLD, dev, sequence_parallel=True)
    torch.manual_seed(0)
    N, K, rows = 384, 512, 256
    w = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    worst = {}
    for kind in ("blockwise", "tensorwise"):
        with FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe(kind)).autocast(True):
            for it in range(3):                        # the site's buffers and flags are reused across calls
                g = torch.Generator(device=dev).manual_seed(100 * it + rank)
                x = (torch.randn(rows, K, device=dev, generator=g) * (1 + rank + it)).bfloat16()
                y = T.ag_gemm_fp8(state, x, [w], "check")
                assert y is not None
                xf = T.all_gather_rows(state, x)
                if kind == "blockwise":
                    a8, sa = fp8.quantize_rowwise(xf)
                    wq, ws, _, _ = fp8._cached_weight(w)
                    ref = fp8.gemm_fp8(a8, sa, wq, ws)
                else:
                    wq, ws, _ = fp8._cached_weight_tensor(w)
                    a8, sa = fp8.quantize_tensor(xf)     # the gathered tensor's maximum = maximum over ranks
                    ref = fp8.gemm_fp8_tensor(a8, sa, wq, ws)
                torch.cuda.synchronize()
                _lib.check_status(dev)
                err = (y.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
                worst[kind] = max(worst.get(kind, 0.0), err)
                exact = xf.float() @ w.float().t()
                rel = ((y.float() - exact).norm() / exact.norm()).item()
                assert rel < 0.07, (kind, it, rel)
    # row-parallel product with the reduce-scatter's send half in the FP8 GEMM epilogue (and the transposed-weight
    # form used for a column-parallel layer's input gradient)
    M = rows * world
    wr = (torch.randn(N, K, device=dev, generator=torch.Generator(device=dev).manual_seed(7 + rank)) * 0.05).bfloat16()
    for kind in ("blockwise", "tensorwise"):
        with FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe(kind)).autocast(True):
            for it in range(3):
                g = torch.Generator(device=dev).manual_seed(1000 + 10 * it + rank)
                xr = torch.randn(M, K, device=dev, generator=g).bfloat16()
                res = torch.randn(rows, N, device=dev, generator=g).bfloat16()
                y = T.gemm_rs_fp8(state, xr, [wr], residual=res)
                assert y is not None
                ref = T.reduce_scatter_rows(state, fp8.forward_product(xr, [wr]).float()) + res.float()
                dyr = torch.randn(M, N, device=dev, generator=g).bfloat16()
                dx = T.gemm_rs_fp8(state, dyr, [wr], transpose_w=True)
                dref = T.reduce_scatter_rows(state, fp8.dgrad_product(dyr, [wr]).float())
                torch.cuda.synchronize()
                _lib.check_status(dev)
                for got, want, tag in ((y, ref, "rs"), (dx, dref, "rs_t")):
                    err = (got.float() - want).abs().max().item() / want.abs().max().item()
                    worst[f"{kind}/{tag}"] = max(worst.get(f"{kind}/{tag}", 0.0), err)
    dist.barrier()
    if rank == 0:
        print("FP8_AG_OK", {k: round(v, 6) for k, v in worst.items()})
    assert all(v < 2e-2 for v in worst.values()), worst
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
