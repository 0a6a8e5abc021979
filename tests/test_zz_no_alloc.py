"""The allocation-free RMSNorm backward must agree with the regular entry point.

Some hosts of this library cannot allocate device memory while they run (all memory belongs to
their own pool, or they are only handed input and output buffers), so one entry point keeps its
scratch inside the library. This test calls it through its exported C symbol, twice in a row
(the built-in scratch is reused and keeps old contents), and compares with ``ob_rmsnorm_bwd``,
which gets its scratch from the caller. It sits last in collection order on purpose.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from optimus_dl_b200.ops import build

    path = build.LIB_PATH if build.LIB_PATH.exists() else build.build()
    lib = ctypes.CDLL(str(path))
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.ob_rmsnorm_bwd_noalloc.argtypes = [P, P, P, P, P, P, I, I, P]
    lib.ob_rmsnorm_bwd_noalloc.restype = I
    lib.ob_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, P]
    lib.ob_rmsnorm_bwd.restype = I
    lib.ob_norm_bwd_grid.argtypes = [I]
    lib.ob_norm_bwd_grid.restype = I
    lib.ob_bind_thread.argtypes = [I]
    lib.ob_bind_thread.restype = I
    return lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("rows,D", [(300, 512), (4096, 4096)])
def test_noalloc_matches_regular_entry_point_twice(rows, D):
    lib = _lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    assert lib.ob_bind_thread(0) == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        torch.manual_seed(call)
        x = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(D, device=dev)).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
        dx_a, dx_b = torch.empty_like(x), torch.empty_like(x)
        dw_a, dw_b = torch.empty(D, device=dev, dtype=torch.bfloat16), torch.empty(D, device=dev, dtype=torch.bfloat16)
        grid = lib.ob_norm_bwd_grid(rows)
        partial = torch.empty(grid * D, device=dev, dtype=torch.float32)
        rc = lib.ob_rmsnorm_bwd(_p(dy), _p(x), _p(w), _p(rstd), None, _p(dx_a), _p(partial), _p(dw_a), None, 0, rows, D,
                                stream)
        assert rc == 0
        rc = lib.ob_rmsnorm_bwd_noalloc(_p(dy), _p(x), _p(w), _p(rstd), _p(dx_b), _p(dw_b), rows, D, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx_a, dx_b), "dx must be identical: same per-row arithmetic"
        ref = dw_a.float()
        err = (dw_b.float() - ref).abs().max().item()
        assert err <= 3e-2 * ref.abs().max().item() + 5e-2, f"call {call}: dw max err {err}"


def test_noalloc_rejects_unsupported_width():
    lib = _lib()
    dev = torch.device("cuda", 0)
    t = torch.zeros(8, device=dev, dtype=torch.bfloat16)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # D beyond the supported width is refused before anything is launched
    assert lib.ob_rmsnorm_bwd_noalloc(_p(t), _p(t), _p(t), _p(t), _p(t), _p(t), 4, 16384, stream) == -1
    assert lib.ob_rmsnorm_bwd_noalloc(_p(t), _p(t), _p(t), _p(t), _p(t), _p(t), 4, 12, stream) == -1
