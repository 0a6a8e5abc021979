"""ctypes loader for the native kernel library (``ops/lib/libob_kernels.so``).

The library is built in-tree by :mod:`optimus_dl_b200.ops.build`. On a machine with a
CUDA device the kernels are mandatory: if the library is missing it is built on the
spot when ``nvcc`` exists, and otherwise loading fails loudly instead of falling back
to eager PyTorch. On CPU-only machines ``available()`` is False and callers use their
PyTorch reference implementations.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import build as _build

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
_status_bufs: dict[int, torch.Tensor] = {}


class KernelError(RuntimeError):
    """A launcher returned a non-zero code or a kernel reported a bounded-wait timeout."""


def available() -> bool:
    return torch.cuda.is_available()


class _CountingLib:
    """Proxy over the CDLL that counts launcher calls (every launcher starts at least one kernel)."""

    def __init__(self, cdll: ctypes.CDLL):
        object.__setattr__(self, "_cdll", cdll)
        object.__setattr__(self, "_wrapped", {})
        object.__setattr__(self, "calls", 0)

    def __getattr__(self, name: str):
        w = self._wrapped.get(name)
        if w is not None:
            return w
        fn = getattr(self._cdll, name)  # AttributeError if the symbol does not exist
        if name in _NO_LAUNCH:
            self._wrapped[name] = fn
            return fn

        def counted(*args, _fn=fn, _self=self):
            if not getattr(_tls, "bound", False):
                # first call into the library from this host thread: bind the CUDA device
                _tls.bound = True
                if torch.cuda.is_available():
                    _self._cdll.ob_bind_thread(torch.cuda.current_device())
            object.__setattr__(_self, "calls", _self.calls + 1)
            if _timeline is not None:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                rc = _fn(*args)
                e.record()
                key = name
                if name == "ob_gemm_bf16":
                    key = f"gemm a_mn={args[2]} b_mn={args[5]} {args[8]}x{args[9]}x{args[10]}"
                _timeline.append((key, s, e))
                return rc
            return _fn(*args)

        self._wrapped[name] = counted
        return counted


_NO_LAUNCH = {"ob_norm_bwd_grid", "ob_rope_grid", "ob_bind_thread", "ob_set_flag_wait_iters", "ob_gemm_skinny_splits",
              "ob_gemm2_ce_tiles"}
_tls = threading.local()


def lib() -> "_CountingLib":
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.LIB_PATH
            if not path.exists():
                path = _build.build()
            cdll = ctypes.CDLL(str(path))
            _declare(cdll)
            _lib = _CountingLib(cdll)
    return _lib


_timeline: list | None = None


def timeline_start() -> None:
    """Start bracketing every launcher call with CUDA events (diagnostics; adds launch overhead)."""
    global _timeline
    _timeline = []


def timeline_report() -> dict[str, tuple[int, float]]:
    """Stop the timeline; returns ``{launcher: (calls, total_ms)}`` measured on the launching stream."""
    global _timeline
    tl, _timeline = _timeline or [], None
    torch.cuda.synchronize()
    out: dict[str, tuple[int, float]] = {}
    for name, s, e in tl:
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + s.elapsed_time(e))
    return out


def launch_count() -> int:
    """Number of kernel-launching calls made into the native library so far."""
    return 0 if _lib is None else _lib.calls


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> c_void_p:
    """The current CUDA stream of the current device as a raw handle (no ``torch.cuda.Stream`` object per launch)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32 word kernels write their error status into (0 = ok)."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    buf = _status_bufs.get(idx)
    if buf is None:
        buf = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_bufs[idx] = buf
    return buf


def check_status(device: torch.device | None = None) -> None:
    """Synchronously read the status word; raise if a kernel reported a timeout."""
    buf = status_word(device)
    code = int(buf.item())
    if code != 0:
        buf.zero_()
        raise KernelError(f"kernel status {code}: {_STATUS_NAMES.get(code, 'unknown')}")


_STATUS_NAMES = {1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad arguments"}


class DeferredStatus:
    """Status word read without stalling the stream: ``post()`` queues a copy of the word to pinned host memory,
    ``check()`` (usually one step later) waits for that copy only and raises if a kernel had reported a failure."""

    def __init__(self, device: torch.device):
        self.device = device
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory() if torch.cuda.is_available() else torch.zeros(1, dtype=torch.int32)
        self.event: torch.cuda.Event | None = None

    def post(self) -> None:
        self.host.copy_(status_word(self.device), non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record()

    def check(self) -> None:
        if self.event is None:
            return
        self.event.synchronize()
        self.event = None
        code = int(self.host[0])
        if code != 0:
            status_word(self.device).zero_()
            raise KernelError(f"kernel status {code}: {_STATUS_NAMES.get(code, 'unknown')} (the optimizer update of that "
                              "step was skipped; parameters and optimizer state are those of the last good step)")


def set_flag_wait_iters(iters: int) -> None:
    """Poll limit of the cross-GPU barrier waits on the current device (0 = default, about two seconds)."""
    check(lib().ob_set_flag_wait_iters(int(iters)), "ob_set_flag_wait_iters")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def _declare(l: ctypes.CDLL) -> None:
    P, I, L, F = c_void_p, c_int, c_longlong, c_float

    def sig(name, args):
        fn = getattr(l, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = c_int

    sig("ob_gemm_bf16", [P, L, I, P, L, I, P, L, I, I, I, I, I, P, I, F, P, I, I, P, I, I, I, I, I, P, P])
    sig("ob_gemm_swiglu_bf16", [P, L, P, P, L, P, P, P, L, I, I, I, P, P])
    sig("ob_gemm_skinny_bf16", [P, L, P, L, P, L, I, I, I, P, I, P, P])
    sig("ob_gemm_skinny_splits", [I, I])
    sig("ob_gemm2_bf16", [P, L, I, P, L, I, P, L, I, I, I, I, I, P, I, F, I, P, P])
    sig("ob_gemm2_swiglu_bf16", [P, L, P, P, L, P, P, P, L, I, I, I, P, P])
    sig("ob_gemm2_swiglu_bwd_bf16", [P, L, P, L, P, P, L, I, I, I, P, P])
    sig("ob_gemm2_ce_tiles", [I])
    sig("ob_gemm2_ce_stats_bf16", [P, L, P, L, I, I, I, P, P, P, P, I, I, F, P, P])
    sig("ob_ce_stats_merge", [P, P, I, I, P, P, P, P, P, I, P])
    sig("ob_rmsnorm_fwd", [P, P, P, P, P, P, I, I, F, P])
    sig("ob_rmsnorm_fwd_fp8", [P, P, P, P, P, P, P, P, L, I, I, F, P])
    sig("ob_rmsnorm_bwd", [P, P, P, P, P, P, P, P, P, I, I, I, P])
    sig("ob_norm_bwd_grid", [I])
    sig("ob_layernorm_fwd", [P, P, P, P, P, P, I, I, F, P])
    sig("ob_layernorm_bwd", [P, P, P, P, P, P, P, P, P, I, I, P])
    sig("ob_rope_grid", [L])
    sig("ob_qknorm_rope_fwd", [P, P, L, L, P, P, P, P, P, I, I, I, I, I, F, P])
    sig("ob_qknorm_rope_bwd", [P, P, L, L, P, L, P, P, P, P, P, P, I, I, I, I, I, P])
    sig("ob_swiglu_fwd", [P, P, P, L, P])
    sig("ob_swiglu_bwd", [P, P, P, P, P, P, L, P])
    sig("ob_adamw", [P, P, P, P, I, P, L, F, F, F, F, F, F, F, F, P, F, P])
    sig("ob_sumsq", [P, L, I, P, P, I, P])
    sig("ob_embedding_fwd", [P, P, P, L, I, I, P])
    sig("ob_embedding_bwd", [P, P, P, P, L, I, I, I, I, P])
    sig("ob_add_f32_to_bf16", [P, P, L, I, P])
    sig("ob_ce_stats", [P, L, P, P, P, P, P, P, P, I, I, I, I, F, P])
    sig("ob_ce_grad", [P, L, P, P, I, I, I, I, L, F, P, F, I, F, P, P])
    sig("ob_attn_fwd", [P, P, P, P, P, P, I, I, I, I, L, L, L, F, I, P, P])
    sig("ob_attn_bwd", [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, L, L, L, F, I, P, P])  # 23 args
    sig("ob_bind_thread", [I])
    PP = ctypes.POINTER(c_void_p)
    sig("ob_barrier", [PP, I, I, I, P, P])
    sig("ob_pull", [P, I, PP, I, P, P, I, I, P])
    sig("ob_rs_adamw", [I, P, I, PP, I, P, P, P, P, P, F, F, F, F, F, F, F, F, P, I, I, P, P])
    sig("ob_set_flag_wait_iters", [ctypes.c_uint])
    sig("ob_gemm_ag_bf16", [P, L, P, L, P, L, I, I, I, P, P, I, PP, I, P, P, I, I, I, I, I, P, P])
    sig("ob_gemm2_ag_bf16", [P, L, P, L, P, L, I, I, I, P, P, I, PP, I, P, P, I, I, I, I, P, P])
    sig("ob_gemm_ag_act_bf16", [P, L, P, P, L, I, P, P, P, L, I, I, I, P, P, I, PP, I, P, P, I, I, I, I, P, P])
    sig("ob_gemm_ag_push_bf16", [P, L, P, L, P, P, L, I, P, P, P, L, I, I, I, P, P, I, PP, PP, I, P, I, I, I, I, P, P])
    sig("ob_gemm_rs_bf16", [P, L, I, P, L, I, P, PP, I, I, I, L, I, I, I, I, P, P])
    sig("ob_gemm_fp8_block", [P, L, P, L, P, L, P, P, L, I, I, I, P, P])
    sig("ob_quant_fp8_rowwise", [P, L, P, L, P, L, I, I, P])
    sig("ob_quant_fp8_block", [P, L, P, L, P, L, P, P, I, I, P, P, P])
    sig("ob_gemm_fp8_tensor", [P, L, P, P, L, P, P, L, I, I, I, I, P, P])
    sig("ob_fp8_amax_scale", [P, L, I, I, P, P, F, P])
    sig("ob_quant_fp8_tensor", [P, L, P, L, P, P, I, I, P])
    sig("ob_gemm_fp8_ag", [P, L, I, PP, PP, L, PP, I, I, I, P, L, P, P, L, I, I, I, P, P, I, P, P])
    sig("ob_gemm_fp8_rs", [P, L, P, L, P, L, P, PP, I, I, I, L, I, I, I, I, I, P, P])
    sig("ob_quant_fp8_tensor_t", [P, L, P, L, P, L, P, P, I, I, P])
    sig("ob_fp8_delayed_update", [P, I, I, I, F, I, P])
    sig("ob_attn_decode", [P, L, P, P, L, P, P, L, L, L, P, P, L, P, P, I, I, I, I, I, I, F, I, P])
    sig("ob_sample", [P, I, L, I, I, F, I, F, I, ctypes.c_uint64, ctypes.c_uint64, P, P])
    sig("ob_embedding_push", [P, I, P, I, I, I, PP, I, I, P])
    sig("ob_rs_sum", [PP, I, I, I, P, I, I, L, P, L, P, L, I, P, P])
