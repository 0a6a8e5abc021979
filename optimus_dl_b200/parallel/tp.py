"""Tensor and sequence parallelism over NVLink peer memory.

The reference shards a model with DTensor plans (optimus_dl/modules/model/llama2.py:215-345,
qwen3.py, olmo3.py): ``wq/wk/wv/w1/w2`` column-wise, ``wo/c_proj`` row-wise, the embedding over
the vocabulary, optionally the norms over the sequence (sequence parallelism) and the head over
the vocabulary with a sharded loss (loss parallelism). The same layouts are produced here, but
the collectives are not separate NCCL calls:

* **all-gather -> column-parallel GEMM** (``csrc/gemm_ag.cu``): copy CTAs pull the peers'
  sequence shards over NVLink while the tensor-core CTAs of the same launch already multiply the
  rows that have landed (per-128-row flags), including the dual-B SwiGLU form;
* **row-parallel GEMM -> reduce-scatter** (``csrc/gemm_core.cuh`` epilogue + ``ob_rs_sum``): the
  epilogue stores each accumulator tile straight into the owning rank's staging slot with peer
  stores; one more kernel does barrier + fixed-order fp32 sum + residual add;
* **vocabulary-parallel embedding**: every rank pushes the rows it owns to the ranks that hold
  the tokens (``ob_embedding_push``), no partial sums are formed at all.

Activations between blocks are ``[tokens / P, D]`` (flattened batch x sequence, contiguous slices
per rank) under sequence parallelism. On CPU, or whenever the CUDA kernels do not apply, every
function falls back to ``torch.distributed`` collectives plus the local op with the same autograd
structure, which is what the Gloo tests exercise.

Buffer reuse: gathered sources and reduce-scatter staging live in two alternating symmetric
buffers each. A rank overwrites buffer ``k`` only after it passed the barrier of use ``k+1``,
which every peer reaches only after finishing its reads of use ``k``.
"""

from __future__ import annotations

import logging
import os
from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _lib, gemm
from ..ops import fp8 as fp8_ops
from ..ops import linear as lin_ops

logger = logging.getLogger(__name__)


class TPState:
    """Everything the tensor-parallel functions need to know about one TP group."""

    def __init__(self, group: Any, device: torch.device, sequence_parallel: bool = False,
                 loss_parallel: bool = False, mesh: Any = None):
        self.group = group
        self.mesh = mesh
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.sequence_parallel = bool(sequence_parallel)
        self.loss_parallel = bool(loss_parallel)
        self.full_shape: tuple[int, int] | None = None  # (B, T) of the running forward
        self.fused = self.device.type == "cuda" and _lib.available()
        self._heap = None
        self._barrier = None
        self._src = [None, None]     # gathered-source ping-pong (symmetric, bf16)
        self._stage = [None, None]   # reduce-scatter staging ping-pong (symmetric, bf16)
        self._src_i = 0
        self._stage_i = 0
        self._flags = None
        self._epoch = 0
        self._tasks: dict = {}
        self.n_copy = 16
        self.n_push = 8              # copy CTAs of the push all-gather (posted stores need few)
        # from this group size on the fused all-gather pushes instead of pulling (the pull
        # form needs no persistent buffers and remains for call sites without a site key); OB_TP_PUSH_MIN_WORLD overrides it
        self.push_min_world = int(os.environ.get("OB_TP_PUSH_MIN_WORLD", "2"))
        self._sites: dict = {}       # persistent gathered-operand buffers, one per call site
        self._push_tasks: dict = {}

    # ------------------------------------------------------------------ symmetric buffers
    def heap(self):
        if self._heap is None:
            from .symm import DeviceBarrier, SymmetricHeap

            self._heap = SymmetricHeap(self.group, self.device)
            self._barrier = DeviceBarrier(self._heap)
        return self._heap

    def barrier(self) -> None:
        self.heap()
        self._barrier()

    def next_barrier_epoch(self) -> int:
        self.heap()
        self._barrier.epoch += 1
        return self._barrier.epoch

    def _grow(self, slots: list, idx: int, numel: int):
        buf = slots[idx]
        if buf is None or buf.tensor.numel() < numel:
            # sizes are a pure function of the model and batch shape, so all ranks grow together
            if buf is not None:
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.group)
            buf = self.heap().empty(numel, torch.bfloat16)
            slots[idx] = buf
        return buf

    def next_src(self, numel: int):
        self._src_i ^= 1
        return self._grow(self._src, self._src_i, numel)

    def next_stage(self, numel: int):
        self._stage_i ^= 1
        return self._grow(self._stage, self._stage_i, numel)

    def flags(self, n: int) -> torch.Tensor:
        if self._flags is None or self._flags.numel() < n:
            self._flags = torch.zeros(max(n, 4096), dtype=torch.int32, device=self.device)
            self._epoch = 0
        return self._flags

    def next_epoch(self) -> int:
        self._epoch += 1
        return self._epoch

    def gather_tasks(self, rows: int, width: int, flag_rows: int):
        """Copy tasks that pull every other rank's ``rows x width`` slice (peers in ring order starting
        after this rank), one task and one flag per ``flag_rows`` rows."""
        key = (rows, width, flag_rows)
        hit = self._tasks.get(key)
        if hit is None:
            from .symm import tasks_to_device

            tasks = []
            per = rows // flag_rows
            for step in range(1, self.size):   # the own slice is copied locally by the caller
                peer = (self.rank + step) % self.size
                for j in range(per):
                    row0 = peer * rows + j * flag_rows
                    tasks.append((row0 * width, flag_rows * width, peer, row0 // flag_rows))
            hit = (tasks_to_device(tasks, self.device), len(tasks))
            self._tasks[key] = hit
        return hit


class _Site:
    """Gathered operand ``[P * rows, width]`` of one call site in symmetric memory plus its row flags. Peers
    store their slices into it (``ob_gemm_ag_push_bf16``); it stays valid until the same site runs again,
    so the backward pass can read the gathered operand without keeping another copy."""

    def __init__(self, tp: "TPState", numel: int, n_flags: int):
        heap = tp.heap()
        self.buf = heap.empty(numel, torch.bfloat16)
        self.flags = heap.empty(max(n_flags, 16), torch.int32, zero=True)
        self.numel, self.n_flags, self.epoch = numel, n_flags, 0
        torch.cuda.synchronize(tp.device)
        dist.barrier(group=tp.group)   # zeroed flags are in place everywhere before anybody publishes into them


class _Fp8Site:
    """Gathered e4m3 operand ``[M, K]``, its 1x128 scale table ``[K / 128, M]`` and row flags of one call site,
    all in symmetric memory: every rank's quantise-and-push CTAs write into every rank's copy
    (``ob_gemm_fp8_ag``)."""

    def __init__(self, tp: "TPState", M: int, K: int):
        heap = tp.heap()
        self.a8 = heap.empty(M * K, torch.uint8)
        self.sa = heap.empty((K // 128) * M, torch.float32)
        self.flags = heap.empty(max(M // 128, 16), torch.int32, zero=True)
        self.M, self.K, self.epoch = M, K, 0
        torch.cuda.synchronize(tp.device)
        dist.barrier(group=tp.group)


def ag_gemm_fp8(tp: "TPState", x_local: torch.Tensor, owners: list, site_key: Any):
    """Quantise this rank's rows, all-gather them in e4m3 and multiply by the (cached) quantised weight in one
    launch. Returns ``y [P * rows, N]`` (bf16), or ``None`` when the shapes do not fit the fused kernel.

    Block recipe: 1x128 scales travel with the rows. Per-tensor recipes: one scale for the gathered tensor, the
    maximum over the group of each rank's own scale (so every rank quantises alike)."""
    rows, K = x_local.shape
    if not (tp.fused and x_local.is_cuda and x_local.dtype == torch.bfloat16 and rows % 128 == 0 and K % 128 == 0
            and K * 4 <= 196608):
        return None
    M = rows * tp.size
    w = owners[0] if len(owners) == 1 else lin_ops._fused_view(list(owners))
    N = w.shape[0]
    x_local = x_local if (x_local.stride(1) == 1 and x_local.stride(0) % 8 == 0) else x_local.contiguous()
    mode = fp8_ops.scaling_mode()
    scale = None
    if mode == "block":
        wq, wscale, _, _ = fp8_ops._cached_weight(w, owners[0])
    else:
        wq, wscale, _ = fp8_ops._cached_weight_tensor(w, owners[0])
        scale = fp8_ops.tensor_scale(x_local, margin_mul=fp8_ops._margin_mul())
        dist.all_reduce(scale, op=dist.ReduceOp.MAX, group=tp.group)
    key = ("fp8", site_key, M, K)
    site = tp._sites.get(key)
    if site is None:
        site = tp._sites[key] = _Fp8Site(tp, M, K)
    site.epoch += 1
    # every rank is done reading this site's previous contents once all ranks have arrived here
    tp.barrier()
    dev = x_local.device
    y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    rc = _lib.lib().ob_gemm_fp8_ag(
        _lib.ptr(x_local), x_local.stride(0), rows, site.a8.peers.c, site.sa.peers.c, M, site.flags.peers.c, tp.size,
        tp.rank, site.epoch, _lib.ptr(wq), wq.stride(0), _lib.ptr(wscale), _lib.ptr(y), N, N, K,
        int(mode != "block"), _lib.ptr(scale), _lib.ptr(None), 2 * tp.n_push, _lib.ptr(_lib.status_word(dev)),
        _lib.stream())
    _lib.check(rc, "ob_gemm_fp8_ag")
    return y


def _site_of(tp: "TPState", key: Any, numel: int, n_flags: int) -> "_Site":
    site = tp._sites.get(key)
    if site is None or site.numel < numel or site.n_flags < n_flags:
        site = _Site(tp, numel, n_flags)
        tp._sites[key] = site
    return site


def _push_tasks_of(tp: "TPState", rows: int, width: int, flag_rows: int):
    """Chunks of this rank's slice for every peer, nearest lower rank first: a receiver then sees the slices of
    ranks me+1, me+2, ... arrive in the order its tiles consume them."""
    key = (rows, width, flag_rows)
    hit = tp._push_tasks.get(key)
    if hit is None:
        from .symm import tasks_to_device

        tasks = []
        per = rows // flag_rows
        for step in range(1, tp.size):
            peer = (tp.rank - step) % tp.size
            for j in range(per):
                row0 = tp.rank * rows + j * flag_rows
                tasks.append((row0 * width, flag_rows * width, peer, row0 // flag_rows))
        hit = (tasks_to_device(tasks, tp.device), len(tasks))
        tp._push_tasks[key] = hit
    return hit


def _flag_rows(rows_per_rank: int) -> int:
    return 128 if rows_per_rank % 128 == 0 else rows_per_rank


def _fusable(tp: TPState, *ts: torch.Tensor) -> bool:
    return tp.fused and all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


# ====================================================================== primitives
def all_gather_rows(tp: TPState, x: torch.Tensor) -> torch.Tensor:
    """``[rows, D]`` per rank -> ``[P * rows, D]`` (rank-major), no autograd."""
    out = torch.empty((x.shape[0] * tp.size, x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=tp.group)
    return out


def reduce_scatter_rows(tp: TPState, x: torch.Tensor) -> torch.Tensor:
    """Sum of every rank's ``[P * rows, D]`` scattered by row block, no autograd."""
    rows = x.shape[0] // tp.size
    if x.device.type == "cpu":  # Gloo has no reduce-scatter
        y = x.contiguous().clone()
        dist.all_reduce(y, group=tp.group)
        return y[tp.rank * rows:(tp.rank + 1) * rows].contiguous()
    out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=tp.group)
    return out


def _publish_rows(tp: TPState, x_local: torch.Tensor):
    """Copy this rank's slice into the next symmetric source buffer and pass the barrier that makes
    every rank's slice readable. Returns ``(buffer, rows, width)``."""
    rows, width = x_local.shape
    buf = tp.next_src(tp.size * rows * width)
    view = buf.tensor[: tp.size * rows * width].view(tp.size * rows, width)
    view[tp.rank * rows:(tp.rank + 1) * rows].copy_(x_local)
    tp.barrier()
    return buf, rows, width


def ag_gemm(tp: TPState, x_local: torch.Tensor, w: torch.Tensor, w2: torch.Tensor | None = None, *,
            b_mn: bool = False, bias: torch.Tensor | None = None, save_gu: bool = False, site: Any = None):
    """Gather ``x`` over the group and multiply in one launch.

    Returns ``(x_full, y)`` or, with ``w2`` (SwiGLU), ``(x_full, h, g, u)``. ``w`` is ``[N, K]``
    (``[K, N]`` with ``b_mn``). With a ``site`` key (any hashable that names the call site) and more than two
    ranks the gather is a push into a persistent symmetric buffer of that site, and ``x_full`` is a view of it
    that stays valid until the site runs again; otherwise slices are pulled into a fresh tensor.
    """
    rows, K = x_local.shape
    M = rows * tp.size
    N = w.shape[1] if b_mn else w.shape[0]
    ok = (_fusable(tp, x_local, w, w2, bias) and K % 8 == 0 and N % 8 == 0 and w.is_contiguous()
          and (w2 is None or (w2.is_contiguous() and w2.shape == w.shape)))
    if not ok:
        x_full = all_gather_rows(tp, x_local)
        if w2 is None:
            return x_full, gemm.gemm(x_full, w, b_mn=b_mn, bias=bias)
        h, g, u = gemm.swiglu_gemm(x_full, w, w2, save_gu=save_gu)
        return x_full, h, g, u
    if site is not None and tp.size >= tp.push_min_world and rows % 128 == 0:
        return _ag_gemm_push(tp, x_local.contiguous(), w, w2, b_mn, bias, save_gu, site)
    buf, _, _ = _publish_rows(tp, x_local.contiguous())
    fr = _flag_rows(rows)
    tasks, n_tasks = tp.gather_tasks(rows, K, fr)
    flags = tp.flags(M // fr + 1)
    epoch = tp.next_epoch()
    x_full = torch.empty((M, K), dtype=torch.bfloat16, device=x_local.device)
    # this rank's rows are in place (and flagged) before the kernel starts: its first tiles never wait
    x_full[tp.rank * rows:(tp.rank + 1) * rows].copy_(x_local)
    flags[(tp.rank * rows) // fr:((tp.rank + 1) * rows + fr - 1) // fr].fill_(epoch)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x_local.device)
    g = u = None
    if w2 is not None and save_gu:
        g = torch.empty_like(y)
        u = torch.empty_like(y)
    rc = _lib.lib().ob_gemm_ag_act_bf16(
        _lib.ptr(x_full), K, _lib.ptr(w), _lib.ptr(w2), w.stride(0), int(b_mn), _lib.ptr(y), _lib.ptr(g), _lib.ptr(u),
        N, M, N, K, _lib.ptr(bias), _lib.ptr(tasks), n_tasks, buf.peers.c, tp.size, _lib.ptr(x_full), _lib.ptr(flags),
        fr, epoch, (tp.rank * rows) // 128, tp.n_copy, _lib.ptr(_lib.status_word(x_local.device)), _lib.stream())
    _lib.check(rc, "ob_gemm_ag_act_bf16")
    if w2 is None:
        return x_full, y
    return x_full, y, g, u


def _ag_gemm_push(tp: TPState, x_local: torch.Tensor, w, w2, b_mn: bool, bias, save_gu: bool, site_key: Any):
    rows, K = x_local.shape
    M = rows * tp.size
    N = w.shape[1] if b_mn else w.shape[0]
    fr = 128
    site = _site_of(tp, (site_key, M, K), M * K, M // fr)
    site.epoch += 1
    x_full = site.buf.tensor[: M * K].view(M, K)
    lo = tp.rank * rows
    x_full[lo:lo + rows].copy_(x_local)
    site.flags.tensor[lo // fr:(lo + rows) // fr].fill_(site.epoch)
    # every rank has finished reading this site's previous contents (its last reader ran before this point in
    # stream order on each rank) once all ranks have arrived here
    tp.barrier()
    tasks, n_tasks = _push_tasks_of(tp, rows, K, fr)
    dev = x_local.device
    y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    g = u = None
    if w2 is not None and save_gu:
        g = torch.empty_like(y)
        u = torch.empty_like(y)
    rc = _lib.lib().ob_gemm_ag_push_bf16(
        _lib.ptr(x_full), K, _lib.ptr(x_local), lo * K, _lib.ptr(w), _lib.ptr(w2), w.stride(0), int(b_mn), _lib.ptr(y),
        _lib.ptr(g), _lib.ptr(u), N, M, N, K, _lib.ptr(bias), _lib.ptr(tasks), n_tasks, site.buf.peers.c,
        site.flags.peers.c, tp.size, _lib.ptr(site.flags.tensor), fr, site.epoch, lo // 128, tp.n_push,
        _lib.ptr(_lib.status_word(dev)), _lib.stream())
    _lib.check(rc, "ob_gemm_ag_push_bf16")
    if w2 is None:
        return x_full, y
    return x_full, y, g, u


def gemm_rs(tp: TPState, a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
            addend: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``reduce_scatter_rows(A B^T + addend) + residual`` with the send half in the GEMM epilogue."""
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    rows = M // tp.size
    ok = (_fusable(tp, a, b, addend, residual) and M % tp.size == 0 and N % 8 == 0 and K % 8 == 0
          and a.is_contiguous() and b.is_contiguous() and (addend is None or addend.is_contiguous())
          and (residual is None or residual.is_contiguous()))
    if not ok:
        y = gemm.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
        if addend is not None:
            y = y + addend
        y = reduce_scatter_rows(tp, y)
        return y if residual is None else y + residual
    stage = tp.next_stage(tp.size * rows * N)
    # send to the next rank's rows first; this rank's own rows last
    shift = (((tp.rank + 1) % tp.size) * rows) // 128
    dev = a.device
    rc = _lib.lib().ob_gemm_rs_bf16(_lib.ptr(a), a.stride(0), int(a_mn), _lib.ptr(b), b.stride(0), int(b_mn),
                                    _lib.ptr(addend), stage.peers.c, tp.size, tp.rank, rows, N, M, N, K, shift,
                                    _lib.ptr(_lib.status_word(dev)), _lib.stream())
    _lib.check(rc, "ob_gemm_rs_bf16")
    out = torch.empty((rows, N), dtype=torch.bfloat16, device=dev)
    epoch = tp.next_barrier_epoch()
    rc = _lib.lib().ob_rs_sum(tp._barrier.buf.peers.c, tp.rank, tp.size, epoch, _lib.ptr(stage.tensor), rows, N, N,
                              _lib.ptr(residual), N, _lib.ptr(out), N, 0, _lib.ptr(_lib.status_word(dev)),
                              _lib.stream())
    _lib.check(rc, "ob_rs_sum")
    return out


def gemm_rs_fp8(tp: TPState, x2: torch.Tensor, owners: list, *, transpose_w: bool = False,
                residual: torch.Tensor | None = None) -> torch.Tensor | None:
    """``reduce_scatter_rows(q(x2) q(W)^T) + residual`` (``q(x2) q(W^T)^T`` with ``transpose_w``: the input gradient
    of a column-parallel layer) with the send half in the FP8 GEMM's epilogue. ``None`` when shapes do not fit."""
    M, K = x2.shape
    rows = M // tp.size
    w = owners[0] if len(owners) == 1 else lin_ops._fused_view(list(owners))
    N = w.shape[1] if transpose_w else w.shape[0]
    if not (tp.fused and x2.is_cuda and x2.dtype == torch.bfloat16 and M % tp.size == 0 and rows % 128 == 0
            and K % 128 == 0 and N % 8 == 0 and (residual is None or residual.is_contiguous())):
        return None
    mode = fp8_ops.scaling_mode()
    if mode == "block":
        wq, ws, wqt, wst = fp8_ops._cached_weight(w, owners[0])
        b8, sb = (wqt, wst) if transpose_w else (wq, ws)
        a8, sa = fp8_ops.quantize_rowwise(x2)
        sa_ld = sa.stride(0)
    else:
        wq, ws, wqt = fp8_ops._cached_weight_tensor(w, owners[0])
        b8, sb = (wqt if transpose_w else wq), ws
        a8, sa = fp8_ops._quantize_activation(x2, owners[0], "dy" if transpose_w else "x")
        sa_ld = 0
    stage = tp.next_stage(tp.size * rows * N)
    shift = (((tp.rank + 1) % tp.size) * rows) // 128   # the next rank's rows first, this rank's own last
    dev = x2.device
    rc = _lib.lib().ob_gemm_fp8_rs(_lib.ptr(a8), a8.stride(0), _lib.ptr(sa), sa_ld, _lib.ptr(b8), b8.stride(0),
                                   _lib.ptr(sb), stage.peers.c, tp.size, tp.rank, rows, N, M, N, K, int(mode != "block"),
                                   shift, _lib.ptr(_lib.status_word(dev)), _lib.stream())
    _lib.check(rc, "ob_gemm_fp8_rs")
    out = torch.empty((rows, N), dtype=torch.bfloat16, device=dev)
    epoch = tp.next_barrier_epoch()
    rc = _lib.lib().ob_rs_sum(tp._barrier.buf.peers.c, tp.rank, tp.size, epoch, _lib.ptr(stage.tensor), rows, N, N,
                              _lib.ptr(residual), N, _lib.ptr(out), N, 0, _lib.ptr(_lib.status_word(dev)),
                              _lib.stream())
    _lib.check(rc, "ob_rs_sum")
    return out


# ====================================================================== autograd functions
def _weight_grads(params: list, dy2: torch.Tensor, x2: torch.Tensor, sizes: list[int], need: list[bool]) -> list:
    """``dW_i = dy_i^T x`` for column slices of ``dy2``; writes into ``main_grad`` where a parameter has one."""
    n = len(params)
    out: list = [None] * n
    mgs = [lin_ops.main_grad_of(p) for p in params]
    if (n > 1 and all(need) and all(m is not None for m in mgs) and lin_ops._adjacent(list(params))
            and lin_ops._adjacent(mgs)):
        accs = [lin_ops.main_grad_write(p) for p in params]
        if all(accs) or not any(accs):
            gemm.gemm(dy2, x2, a_mn=True, b_mn=True, out=lin_ops._fused_view(mgs), accumulate=accs[0])
            return out
        o = 0  # mixed state: per-weight writes
        for p, m, s, a in zip(params, mgs, sizes, accs):
            gemm.gemm(dy2[:, o:o + s], x2, a_mn=True, b_mn=True, out=m, accumulate=a)
            o += s
        return out
    o = 0
    for i, (p, m, s) in enumerate(zip(params, mgs, sizes)):
        if need[i]:
            if m is not None:
                gemm.gemm(dy2[:, o:o + s], x2, a_mn=True, b_mn=True, out=m, accumulate=lin_ops.main_grad_write(p))
            else:
                out[i] = gemm.gemm(dy2[:, o:o + s], x2, a_mn=True, b_mn=True)
        o += s
    return out


def _cat_weights(ws: list[torch.Tensor]) -> torch.Tensor:
    if len(ws) == 1:
        return ws[0]
    if lin_ops._adjacent(ws):
        return lin_ops._fused_view(ws)
    return torch.cat(ws, dim=0)


class _ColumnParallel(torch.autograd.Function):
    """``y = X cat(W_i)^T + b`` with ``W_i`` holding this rank's output rows.

    Sequence-parallel: ``X`` is the all-gather of the per-rank token slices (fused into the GEMM);
    the input gradient is reduce-scattered from the dgrad GEMM's epilogue. Otherwise ``X`` is
    replicated and the input gradient is all-reduced.
    """

    @staticmethod
    def forward(ctx, tp: TPState, sp: bool, x, n, *wb):
        ws, bs = list(wb[:n]), list(wb[n:])
        lin_ops.ensure_gathered(ws)   # a sharding engine may still be gathering these weights
        bias = None if bs[0] is None else lin_ops._fused_bias(bs)
        wf = _cat_weights(ws)
        use_fp8 = fp8_ops.usable(x, ws)
        regather = False
        if use_fp8:
            y = ag_gemm_fp8(tp, x, ws, ("col", id(ws[0]))) if sp else None
            if y is not None:
                # fused quantise + e4m3 all-gather + GEMM; the bf16 rows are gathered again for the weight gradient
                x_full, regather = x, True
            else:
                x_full = all_gather_rows(tp, x) if sp else x
                y = fp8_ops.forward_product(x_full, ws)
            if bias is not None:
                y = y + bias
        elif sp:
            x_full, y = ag_gemm(tp, x, wf, bias=bias, site=("col", id(ws[0])))
        else:
            x_full, y = x, gemm.gemm(x, wf, bias=bias)
        ctx.save_for_backward(x_full, *ws)
        ctx.use_fp8, ctx.regather = use_fp8, regather
        ctx.tp, ctx.sp, ctx.n, ctx.params, ctx.has_bias = tp, sp, n, ws, bias is not None
        ctx.sizes = [w.shape[0] for w in ws]
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, *ws = ctx.saved_tensors
        tp, n = ctx.tp, ctx.n
        if ctx.regather:
            x_full = all_gather_rows(tp, x_full)
        dy2 = dy if dy.is_contiguous() else dy.contiguous()
        wf = _cat_weights(ws)
        dx = None
        if ctx.needs_input_grad[2]:
            if ctx.use_fp8:
                dx = gemm_rs_fp8(tp, dy2, ctx.params, transpose_w=True) if ctx.sp else None
                if dx is None:
                    dx = fp8_ops.dgrad_product(dy2, ctx.params)
                    if ctx.sp:
                        dx = reduce_scatter_rows(tp, dx)
                    else:
                        dist.all_reduce(dx, group=tp.group)
            elif ctx.sp:
                dx = gemm_rs(tp, dy2, wf, b_mn=True)
            else:
                dx = gemm.gemm(dy2, wf, b_mn=True)
                dist.all_reduce(dx, group=tp.group)
        dws = _weight_grads(ctx.params, dy2, x_full, ctx.sizes, [ctx.needs_input_grad[4 + i] for i in range(n)])
        dbs: list = [None] * n
        if ctx.has_bias:
            db = dy2.float().sum(0).to(dy.dtype)
            o = 0
            for i, s in enumerate(ctx.sizes):
                dbs[i] = db[o:o + s]
                o += s
        return (None, None, dx, None, *dws, *dbs)


class _ColumnParallelSwiGLU(torch.autograd.Function):
    """``h = silu(X W1^T) * (X W2^T)`` with column-sharded ``W1, W2``; gathers ``X`` inside the dual-B GEMM."""

    @staticmethod
    def forward(ctx, tp: TPState, sp: bool, x, w1, w2):
        if sp:
            x_full, h, g, u = ag_gemm(tp, x, w1, w2, save_gu=True, site=("glu", id(w1)))
        else:
            x_full = x
            h, g, u = gemm.swiglu_gemm(x, w1, w2, save_gu=True)
        ctx.save_for_backward(x_full, w1, w2, g, u)
        ctx.tp, ctx.sp, ctx.params = tp, sp, (w1, w2)
        return h

    @staticmethod
    def backward(ctx, dh):
        from ..ops.activation import swiglu_backward

        x_full, w1, w2, g, u = ctx.saved_tensors
        tp = ctx.tp
        dg, du = swiglu_backward(dh if dh.is_contiguous() else dh.contiguous(), g, u)
        dx = None
        if ctx.needs_input_grad[2]:
            part = gemm.gemm(dg, w1, b_mn=True)
            if ctx.sp:
                dx = gemm_rs(tp, du, w2, b_mn=True, addend=part)
            else:
                dx = gemm.gemm(du, w2, b_mn=True, out=part, accumulate=True)
                dist.all_reduce(dx, group=tp.group)
        d1 = _weight_grads([ctx.params[0]], dg, x_full, [w1.shape[0]], [ctx.needs_input_grad[3]])[0]
        d2 = _weight_grads([ctx.params[1]], du, x_full, [w2.shape[0]], [ctx.needs_input_grad[4]])[0]
        return None, None, dx, d1, d2


class _RowParallel(torch.autograd.Function):
    """``y = reduce(X_r W_r^T) + b + residual`` with ``W_r`` holding this rank's input columns.

    Sequence-parallel: the reduction is a reduce-scatter over tokens whose send half is the GEMM
    epilogue; in the backward the gradient's all-gather is fused into the dgrad GEMM.
    """

    @staticmethod
    def forward(ctx, tp: TPState, sp: bool, x, w, bias, residual):
        use_fp8 = fp8_ops.usable(x, [w])
        ctx.use_fp8 = use_fp8
        if use_fp8:
            xc = x if x.is_contiguous() else x.contiguous()
            y = gemm_rs_fp8(tp, xc, [w], residual=residual) if sp else None
            if y is None:
                y = fp8_ops.forward_product(xc, [w])
                if sp:
                    y = reduce_scatter_rows(tp, y)
                else:
                    dist.all_reduce(y, group=tp.group)
                if residual is not None:
                    y = y + residual
            if bias is not None:
                y = y + bias
        elif sp:
            y = gemm_rs(tp, x, w, residual=residual)
            if bias is not None:
                y = y + bias
        else:
            y = gemm.gemm(x, w)
            dist.all_reduce(y, group=tp.group)
            if bias is not None:
                y = y + bias
            if residual is not None:
                y = y + residual
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.sp, ctx.param, ctx.has_bias = tp, sp, w, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy2 = dy if dy.is_contiguous() else dy.contiguous()
        if ctx.use_fp8:
            dy_full = all_gather_rows(tp, dy2) if ctx.sp else dy2
            dx = fp8_ops.dgrad_product(dy_full, [ctx.param])
        elif ctx.sp:
            dy_full, dx = ag_gemm(tp, dy2, w, b_mn=True, site=("row_bwd", id(ctx.param)))
        else:
            dy_full, dx = dy2, gemm.gemm(dy2, w, b_mn=True)
        dw = _weight_grads([ctx.param], dy_full, x, [w.shape[0]], [ctx.needs_input_grad[3]])[0]
        db = dy2.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        dres = dy if ctx.needs_input_grad[5] else None
        return None, None, dx, dw, db, dres


class _GatherRows(torch.autograd.Function):
    """All-gather of token slices. ``reduce_grad``: the incoming gradient is a per-rank partial and
    is reduce-scattered; otherwise it is already complete and only sliced."""

    @staticmethod
    def forward(ctx, tp: TPState, x, reduce_grad: bool):
        ctx.tp, ctx.reduce_grad, ctx.rows = tp, reduce_grad, x.shape[0]
        return all_gather_rows(tp, x)

    @staticmethod
    def backward(ctx, dy):
        tp = ctx.tp
        if ctx.reduce_grad:
            return None, reduce_scatter_rows(tp, dy), None
        return None, dy[tp.rank * ctx.rows:(tp.rank + 1) * ctx.rows].contiguous(), None


class _GatherCols(torch.autograd.Function):
    """All-gather along the last dimension (sharded logits -> full logits)."""

    @staticmethod
    def forward(ctx, tp: TPState, x):
        ctx.tp, ctx.cols = tp, x.shape[-1]
        parts = [torch.empty_like(x) for _ in range(tp.size)]
        dist.all_gather(parts, x.contiguous(), group=tp.group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, dy):
        tp = ctx.tp
        return None, dy[..., tp.rank * ctx.cols:(tp.rank + 1) * ctx.cols].contiguous()


class _CopyToGroup(torch.autograd.Function):
    """Identity whose gradient is summed over the group (input of a replicated-input sharded op)."""

    @staticmethod
    def forward(ctx, tp: TPState, x):
        ctx.tp = tp
        return x

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous().clone()
        dist.all_reduce(dy, group=ctx.tp.group)
        return None, dy


class _VocabParallelEmbedding(torch.autograd.Function):
    """Embedding whose table rows are sharded over the group (``RowwiseParallel`` on ``wte``).

    Sequence-parallel + CUDA: each rank stores the rows it owns straight into the token owner's
    activation buffer over NVLink (``ob_embedding_push``), then one barrier. Otherwise: masked
    local lookup followed by a reduce-scatter (sequence-parallel) or all-reduce.
    """

    @staticmethod
    def forward(ctx, tp: TPState, sp: bool, ids, table, pad_id):
        ids64 = ids.reshape(-1).to(torch.int64).contiguous()
        T = ids64.numel()
        v_local, D = table.shape
        voff = tp.rank * v_local
        ctx.save_for_backward(ids64)
        ctx.tp, ctx.sp, ctx.table, ctx.pad_id = tp, sp, table, pad_id
        if sp and _fusable(tp, table) and T % tp.size == 0 and D % 8 == 0 and table.is_contiguous():
            rows = T // tp.size
            buf = tp.next_src(rows * D)
            rc = _lib.lib().ob_embedding_push(_lib.ptr(ids64), T, _lib.ptr(table), v_local, voff, D, buf.peers.c,
                                              tp.size, rows, _lib.stream())
            _lib.check(rc, "ob_embedding_push")
            tp.barrier()
            return buf.tensor[: rows * D].view(rows, D).clone()
        local = ids64 - voff
        mask = (local >= 0) & (local < v_local)
        part = torch.nn.functional.embedding(local.clamp(0, v_local - 1), table) * mask.unsqueeze(-1).to(table.dtype)
        if sp:
            return reduce_scatter_rows(tp, part)
        dist.all_reduce(part, group=tp.group)
        return part

    @staticmethod
    def backward(ctx, dout):
        (ids64,) = ctx.saved_tensors
        tp, table = ctx.tp, ctx.table
        v_local, D = table.shape
        voff = tp.rank * v_local
        d2 = dout.reshape(-1, D).contiguous()
        if ctx.sp:
            d2 = all_gather_rows(tp, d2)
        local = ids64 - voff
        pad = -1
        if ctx.pad_id is not None and 0 <= int(ctx.pad_id) - voff < v_local:
            pad = int(ctx.pad_id) - voff
        if d2.is_cuda and d2.dtype == torch.bfloat16 and _lib.available():
            sorted_ids, perm = torch.sort(local, stable=True)
            mg = lin_ops.main_grad_of(table)
            if mg is not None:
                if not getattr(table, "_main_grad_filled", False):
                    mg.zero_()
                    table._main_grad_filled = True
                dtable, acc, ret = mg, 1, None
            else:
                dtable = torch.zeros((v_local, D), dtype=d2.dtype, device=d2.device)
                acc, ret = 0, dtable
            _lib.check(_lib.lib().ob_embedding_bwd(_lib.ptr(sorted_ids), _lib.ptr(perm), _lib.ptr(d2), _lib.ptr(dtable),
                                                   local.numel(), D, v_local, pad, acc, _lib.stream()),
                       "ob_embedding_bwd")
            return None, None, None, ret, None
        mask = (local >= 0) & (local < v_local) & (local != pad)
        dtable = torch.zeros((v_local, D), dtype=torch.float32, device=d2.device)
        dtable.index_add_(0, local[mask], d2[mask].float())
        return None, None, None, dtable.to(table.dtype), None


# ====================================================================== functional API used by the blocks
def column_parallel_linear(tp: TPState, x: torch.Tensor, weights: list[torch.Tensor], biases: list | None = None):
    """``x`` is ``[rows, D]`` (token slice under sequence parallelism, all tokens otherwise)."""
    n = len(weights)
    biases = list(biases) if biases is not None else [None] * n
    if any(b is None for b in biases):
        biases = [None] * n
    return _ColumnParallel.apply(tp, tp.sequence_parallel, x, n, *weights, *biases)


def row_parallel_linear(tp: TPState, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                        residual: torch.Tensor | None = None) -> torch.Tensor:
    return _RowParallel.apply(tp, tp.sequence_parallel, x, weight, bias, residual)


def column_parallel_swiglu(tp: TPState, x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    return _ColumnParallelSwiGLU.apply(tp, tp.sequence_parallel, x, w1, w2)


def vocab_parallel_embedding(tp: TPState, ids: torch.Tensor, table: torch.Tensor, pad_id: int | None) -> torch.Tensor:
    return _VocabParallelEmbedding.apply(tp, tp.sequence_parallel, ids, table, pad_id)


def gather_tokens(tp: TPState, x: torch.Tensor, grad_is_partial: bool) -> torch.Tensor:
    """Token slices ``[rows, D]`` -> all tokens; identity without sequence parallelism (then a
    partial gradient is all-reduced instead)."""
    if tp.sequence_parallel:
        return _GatherRows.apply(tp, x, grad_is_partial)
    return _CopyToGroup.apply(tp, x) if grad_is_partial else x


def gather_vocab(tp: TPState, logits: torch.Tensor) -> torch.Tensor:
    return _GatherCols.apply(tp, logits)


class _ShardedRMSNorm(torch.autograd.Function):
    """RMSNorm over a feature dimension that is split across the group (full-width QK-norm of
    OLMo-3 under tensor parallelism): the mean of squares is all-reduced, the weight is sharded."""

    @staticmethod
    def forward(ctx, tp: TPState, x, w, eps: float):
        xf = x.float()
        ss = xf.pow(2).sum(-1, keepdim=True)
        dist.all_reduce(ss, group=tp.group)
        n_total = x.shape[-1] * tp.size
        rstd = torch.rsqrt(ss / n_total + eps)
        ctx.save_for_backward(x, w, rstd)
        ctx.tp, ctx.n_total = tp, n_total
        return (xf * rstd * w.float()).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        xf, g = x.float(), dy.float() * w.float()
        dot = (g * xf).sum(-1, keepdim=True)
        dist.all_reduce(dot, group=ctx.tp.group)
        dx = g * rstd - xf * (rstd.pow(3) * dot / ctx.n_total)
        dw = (dy.float() * xf * rstd).reshape(-1, x.shape[-1]).sum(0)
        return None, dx.to(x.dtype), dw.to(w.dtype), None


# ====================================================================== block-level forwards
def attention_forward(mod: nn.Module, x: torch.Tensor, *, freqs_cis=None, position_ids=None, doc_start=None):
    """Tensor-parallel forward of ``models.blocks.attention.BaseSelfAttention`` (local heads only)."""
    from ..ops import attention as attn_ops

    tp: TPState = mod.tp
    B, T = tp.full_shape
    D = x.shape[-1]
    qkv = column_parallel_linear(tp, x.reshape(-1, D), [mod.wq.weight, mod.wk.weight, mod.wv.weight],
                                 [mod.wq.bias, mod.wk.bias, mod.wv.bias])
    Hq, Hk, hd = mod.n_head, mod.n_kv_head, mod.head_dim  # local counts (set by apply_tensor_parallel)
    qkv = qkv.view(B, T, (Hq + 2 * Hk) * hd)
    qw = kw = None
    if mod.use_qk_norm:
        if mod.qk_norm_per_head:
            qw, kw = mod.q_norm.weight, mod.k_norm.weight
        else:
            q, k, v = qkv.split([Hq * hd, Hk * hd, Hk * hd], dim=-1)
            q = _ShardedRMSNorm.apply(tp, q, mod.q_norm.weight, mod.rmsnorm_eps)
            k = _ShardedRMSNorm.apply(tp, k, mod.k_norm.weight, mod.rmsnorm_eps)
            qkv = torch.cat([q, k, v], dim=-1)
    y = attn_ops.qkv_attention(qkv, n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=doc_start,
                               freqs_cis=freqs_cis if mod.use_rope else None,
                               position_ids=position_ids if mod.use_rope else None, q_norm_weight=qw,
                               k_norm_weight=kw, norm_eps=mod.rmsnorm_eps, window=mod.sliding_window,
                               dropout_p=mod.attn_dropout.p if mod.training else 0.0)
    out = row_parallel_linear(tp, y.reshape(B * T, Hq * hd), mod.wo.weight, mod.wo.bias)
    out = out.view(1, -1, D) if tp.sequence_parallel else out.view(B, T, D)
    return mod.resid_dropout(out) if mod.training and mod.resid_dropout.p > 0 else out


def swiglu_mlp_forward(mod: nn.Module, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-parallel forward of ``models.blocks.mlp.SwiGLUMLP`` (gate/up column-, down row-sharded)."""
    from ..ops import activation as act_ops

    tp: TPState = mod.tp
    shp = x.shape
    x2 = x.reshape(-1, shp[-1])
    if mod.w1.bias is None and not lin_ops.fp8_route([mod.w1.weight, mod.w2.weight]):
        h = column_parallel_swiglu(tp, x2, mod.w1.weight, mod.w2.weight)
    else:
        gu = column_parallel_linear(tp, x2, [mod.w1.weight, mod.w2.weight], [mod.w1.bias, mod.w2.bias])
        g, u = gu.split(mod.w1.weight.shape[0], dim=-1)   # also the FP8 form: gate/up as one block-scaled GEMM
        h = act_ops.swiglu(g.contiguous(), u.contiguous())
    res2 = residual.reshape(-1, shp[-1]) if residual is not None else None
    y = row_parallel_linear(tp, h, mod.c_proj.weight, mod.c_proj.bias, residual=res2).view(shp)
    return mod.dropout(y) if mod.dropout is not None else y


def dense_mlp_forward(mod: nn.Module, x: torch.Tensor, act, residual: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-parallel forward of the ``c_fc -> act -> c_proj`` feed-forward blocks."""
    tp: TPState = mod.tp
    shp = x.shape
    h = act(column_parallel_linear(tp, x.reshape(-1, shp[-1]), [mod.c_fc.weight], [mod.c_fc.bias]))
    res2 = residual.reshape(-1, shp[-1]) if residual is not None else None
    y = row_parallel_linear(tp, h, mod.c_proj.weight, mod.c_proj.bias, residual=res2).view(shp)
    return mod.dropout(y) if mod.dropout is not None else y


def embed_forward(model: nn.Module, input_ids: torch.Tensor) -> torch.Tensor:
    tp: TPState = model._tp
    B, T = input_ids.shape
    wte = model.transformer.wte
    x = vocab_parallel_embedding(tp, input_ids, wte.weight, wte.padding_idx)
    D = x.shape[-1]
    return x.view(1, -1, D) if tp.sequence_parallel else x.view(B, T, D)


def hidden_forward(model: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """Final hidden states for the fused head+loss path: all tokens on every rank. The loss
    kernels all-reduce the hidden gradient themselves, so the gather's backward only slices."""
    tp: TPState = model._tp
    B, T = tp.full_shape
    D = x.shape[-1]
    return gather_tokens(tp, x.reshape(-1, D), grad_is_partial=False).view(B, T, D)


def head_forward(model: nn.Module, x: torch.Tensor) -> torch.Tensor:
    """Logits from the vocabulary-sharded head, gathered to the full vocabulary."""
    tp: TPState = model._tp
    B, T = tp.full_shape
    D = x.shape[-1]
    local = column_parallel_linear(tp, x.reshape(-1, D), [model.lm_head.weight], [model.lm_head.bias])
    return gather_vocab(tp, local).view(B, T, -1)


# ====================================================================== applying the plan
def _group_of(mesh: Any):
    if mesh is None:
        return dist.group.WORLD
    if hasattr(mesh, "get_group"):
        return mesh.get_group()
    return mesh  # already a process group


def _shard_param(p: torch.Tensor, dim: int, rank: int, size: int, device: torch.device, out: torch.Tensor | None = None):
    n = p.shape[dim]
    assert n % size == 0, f"dimension {dim} of size {n} is not divisible by the tensor-parallel size {size}"
    piece = p.detach().narrow(dim, rank * (n // size), n // size)
    if out is not None:
        out.copy_(piece)
        return out
    return piece.to(device).contiguous().clone()


def _mark(p: nn.Parameter, tp: TPState, dim: int | None, partial_grad: bool = False) -> nn.Parameter:
    p._tp_shard_dim = dim          # None = replicated over the group
    p._tp_state = tp
    if partial_grad and tp.size > 1 and not getattr(p, "_tp_hooked", False):
        # replicated parameter whose gradient is computed from this rank's tokens / heads only
        p._tp_hooked = True
        group = tp.group

        def _sync(param, group=group):
            if param.grad is not None:
                dist.all_reduce(param.grad, group=group)

        p.register_post_accumulate_grad_hook(_sync)
    return p


def _shard_linears_adjacent(mods: list[nn.Linear], dim: int, tp: TPState) -> None:
    """Replace the weights (and biases for column sharding) of ``mods`` by this rank's shards,
    laid out back to back in one buffer so that sibling projections run as one GEMM."""
    dev, r, P = tp.device, tp.rank, tp.size
    shapes = []
    for m in mods:
        shp = list(m.weight.shape)
        shp[dim] //= P
        shapes.append(shp)
    dtype = mods[0].weight.dtype
    flat = torch.empty(sum(s[0] * s[1] for s in shapes), dtype=dtype, device=dev)
    o = 0
    for m, shp in zip(mods, shapes):
        view = flat[o:o + shp[0] * shp[1]].view(shp)
        _shard_param(m.weight, dim, r, P, dev, out=view)
        req = m.weight.requires_grad
        marked_fp8 = bool(getattr(m.weight, "_fp8", False))
        m.weight = _mark(nn.Parameter(view, requires_grad=req), tp, dim)
        if marked_fp8:
            m.weight._fp8 = True   # the FP8 mark of the transformer_engine transform survives the re-sharding
        o += shp[0] * shp[1]
        if dim == 0:
            m.out_features = shp[0]
        else:
            m.in_features = shp[1]
    if mods[0].bias is not None:
        if dim == 0:
            sizes = [s[0] for s in shapes]
            bflat = torch.empty(sum(sizes), dtype=mods[0].bias.dtype, device=dev)
            o = 0
            for m, s in zip(mods, sizes):
                view = bflat[o:o + s]
                _shard_param(m.bias, 0, r, P, dev, out=view)
                m.bias = _mark(nn.Parameter(view, requires_grad=m.bias.requires_grad), tp, 0)
                o += s
        else:
            for m in mods:
                m.bias = _mark(nn.Parameter(m.bias.detach().to(dev).clone(), requires_grad=m.bias.requires_grad), tp,
                               None, partial_grad=tp.sequence_parallel)


def apply_tensor_parallel(model: nn.Module, mesh: Any, loss_parallel: bool = False, sequence_parallel: bool = False,
                          device: torch.device | str | None = None) -> nn.Module:
    """Shard ``model`` (Llama / Qwen-3 / OLMo-3 layouts) over the tensor-parallel ``mesh`` in place.

    Same plan as the reference's ``apply_tp`` (optimus_dl/modules/model/llama2.py:215-345):
    ``wte`` by vocabulary rows, ``wq/wk/wv`` and the MLP's up projections by output rows, ``wo`` and
    ``c_proj`` by input columns, ``lm_head`` by vocabulary rows; with ``sequence_parallel`` the
    residual stream and the norms work on ``tokens / P`` per rank. Parameters are moved to the
    tensor-parallel device while they are cut, so sibling shards stay adjacent in memory.
    """
    group = _group_of(mesh)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    tp = TPState(group, torch.device(device), sequence_parallel=sequence_parallel, loss_parallel=loss_parallel,
                 mesh=mesh if hasattr(mesh, "get_group") else None)
    P = tp.size
    cfg = model.config
    n_kv = cfg.n_kv_head if getattr(cfg, "n_kv_head", None) is not None else cfg.n_head
    assert cfg.n_head % P == 0, f"Number of heads ({cfg.n_head}) must be divisible by TP size ({P})"
    assert n_kv % P == 0, f"Number of KV heads ({n_kv}) must be divisible by TP size ({P})"
    assert cfg.vocab_size % P == 0, f"vocab_size ({cfg.vocab_size}) must be divisible by TP size ({P})"
    tied = model.transformer.wte.weight is model.lm_head.weight
    model.to(tp.device)
    sp = sequence_parallel
    for m in model.modules():
        if getattr(m, "_fp8_out", False):
            m._fp8_out = False   # under TP the fused all-gather kernel quantises; a norm-side copy would go unused
    for block in model.transformer.h:
        attn = block.attn
        _shard_linears_adjacent([attn.wq, attn.wk, attn.wv], 0, tp)
        _shard_linears_adjacent([attn.wo], 1, tp)
        attn.n_head //= P
        attn.n_kv_head //= P
        attn.tp = tp
        if attn.use_qk_norm:
            for nm in (attn.q_norm, attn.k_norm):
                if attn.qk_norm_per_head:
                    _mark(nm.weight, tp, None, partial_grad=True)
                else:
                    w = _shard_param(nm.weight, 0, tp.rank, P, tp.device)
                    nm.weight = _mark(nn.Parameter(w, requires_grad=nm.weight.requires_grad), tp, 0)
        mlp = block.mlp
        if hasattr(mlp, "w1"):
            _shard_linears_adjacent([mlp.w1, mlp.w2], 0, tp)
        else:
            _shard_linears_adjacent([mlp.c_fc], 0, tp)
        _shard_linears_adjacent([mlp.c_proj], 1, tp)
        mlp.tp = tp
        for name, sub in block.named_children():
            if name not in ("attn", "mlp"):
                for p in sub.parameters(recurse=True):
                    _mark(p, tp, None, partial_grad=sp)
    for p in model.transformer.ln_f.parameters():
        _mark(p, tp, None, partial_grad=sp)
    head_w = _shard_param(model.lm_head.weight, 0, tp.rank, P, tp.device)
    model.lm_head.weight = _mark(nn.Parameter(head_w, requires_grad=model.lm_head.weight.requires_grad), tp, 0)
    model.lm_head.out_features = head_w.shape[0]
    if tied:
        model.transformer.wte.weight = model.lm_head.weight
    else:
        wte = model.transformer.wte
        w = _shard_param(wte.weight, 0, tp.rank, P, tp.device)
        wte.weight = _mark(nn.Parameter(w, requires_grad=wte.weight.requires_grad), tp, 0)
    model.transformer.wte.num_embeddings = model.lm_head.weight.shape[0]
    model._tp = tp
    # the fused head + loss path reads this (criterion/cross_entropy.py: head_parallel_info)
    model._vocab_parallel = {"group": group, "offset": tp.rank * head_w.shape[0], "total": cfg.vocab_size}
    return model
