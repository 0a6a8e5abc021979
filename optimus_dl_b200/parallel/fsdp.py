"""Fully-sharded data parallelism built on flat symmetric buffers and this package's own kernels.

Semantics follow FSDP2 as the reference uses it (optimus_dl/modules/model_transforms/
distributed.py:187-332; per-model grouping in optimus_dl/modules/model/gpt2.py:325-338):
one parameter group per transformer block plus a root group (embeddings, final norm, head);
every parameter is sharded along dim 0 across the shard group; parameters are computed in bf16
while each rank keeps fp32 master weights and optimizer state for its shard only; gradients are
averaged over the data-parallel ranks; ``reshard_after_forward=False`` (the reference default)
keeps gathered parameters until the step ends.

What differs is the mechanism, which is built for NVLink peer access instead of NCCL:

* Each group owns two *symmetric* flat bf16 buffers, parameters and gradients, laid out
  parameter-major (every parameter is contiguous and complete), so sibling projections can be
  fused into one GEMM by viewing adjacent parameters as one matrix (``ops/linear.py``).
* all-gather = peers *pull* the owner's rows straight into place (``ob_pull``); for a block the
  rows of the fused QKV weight are pulled by copy CTAs inside the QKV GEMM launch itself, which
  waits per row group (``ob_gemm_ag_bf16``), and the rest of the block is prefetched one block
  ahead on a side stream.
* reduce-scatter = the owner pulls its rows of every peer's gradient buffer, adds them in a fixed
  rank order in fp32, and applies AdamW to its fp32 shard in the same kernel, writing the new
  bf16 values into its rows of the parameter buffer (``ob_rs_adamw``). With gradient clipping the
  kernel runs in two phases (reduce + squared norm, then update with the clip factor).
* Cross-GPU ordering uses a bounded flag barrier (``parallel/symm.DeviceBarrier``).

A world of one runs the same code (the peer list is the local pointer), which is how the
single-GPU benchmark exercises the identical kernels.
"""

from __future__ import annotations

import logging
import math
from dataclasses import dataclass, field
from typing import Any, Iterable

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _lib
from ..ops import optim as optim_ops
from . import symm

logger = logging.getLogger(__name__)

ALIGN = 8          # elements: 16 bytes of bf16, the vector width of the copy / update kernels
FLAG_ROWS = 128    # rows of the gathered QKV weight guarded by one readiness flag


@dataclass
class ParamInfo:
    name: str
    param: nn.Parameter
    shape: tuple
    rows: int
    row_numel: int
    piece_rows: int        # rows owned by each rank (dim 0 padded up to a multiple of world)
    flat_off: int          # element offset of the parameter in the flat buffers
    shard_off: int = 0     # element offset of this rank's piece in the fp32 shard state
    weight_decay: float = 0.0
    lr_scale: float = 1.0

    @property
    def piece_numel(self) -> int:
        return self.piece_rows * self.row_numel

    @property
    def padded_numel(self) -> int:
        return self.piece_numel * 1  # per rank; total = piece_numel * world


class ShardGroup:
    """One sharding unit: flat symmetric parameter / gradient buffers and this rank's fp32 shard."""

    def __init__(self, name: str, named_params: list[tuple[str, nn.Parameter]], heap: symm.SymmetricHeap,
                 device: torch.device, first_gemm_params: list[nn.Parameter] | None = None):
        self.name = name
        self.heap = heap
        self.device = device
        self.world, self.rank = heap.world, heap.rank
        W = self.world
        self.infos: list[ParamInfo] = []
        off = 0
        # the parameters consumed by the group's first GEMM go first and back to back
        first_ids = [id(p) for p in (first_gemm_params or [])]
        ordered = sorted(named_params, key=lambda np_: (first_ids.index(id(np_[1])) if id(np_[1]) in first_ids else len(first_ids)))
        for pname, p in ordered:
            shape = tuple(p.shape)
            rows = shape[0] if len(shape) > 0 else 1
            row_numel = max(1, p.numel() // max(rows, 1))
            piece_rows = math.ceil(rows / W)
            off = (off + ALIGN - 1) // ALIGN * ALIGN
            self.infos.append(ParamInfo(pname, p, shape, rows, row_numel, piece_rows, off))
            off += piece_rows * W * row_numel
        self.flat_numel = (off + ALIGN - 1) // ALIGN * ALIGN
        soff = 0
        for inf in self.infos:
            soff = (soff + 3) // 4 * 4
            inf.shard_off = soff
            soff += inf.piece_numel
        self.shard_numel = (soff + 3) // 4 * 4
        self.param_buf = heap.empty(self.flat_numel, torch.bfloat16, zero=True)
        self.grad_buf = heap.empty(self.flat_numel, torch.bfloat16, zero=True)
        self.flat_param = self.param_buf.tensor
        self.flat_grad = self.grad_buf.tensor
        self.master = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        self.exp_avg: torch.Tensor | None = None
        self.exp_avg_sq: torch.Tensor | None = None
        self.grad_shard: torch.Tensor | None = None
        self.first_gemm_infos = [inf for inf in self.infos if id(inf.param) in first_ids]
        self._adopt_parameters()
        self._build_tables()
        self.gathered = self.world == 1
        self.rest_event: torch.cuda.Event | None = None
        self.grads_reduced = False
        self.updated_in_backward = False

    # ---------------------------------------------------------------- construction
    def _adopt_parameters(self) -> None:
        """Move parameter storage into the flat buffer; keep fp32 masters of the owned rows."""
        for inf in self.infos:
            p = inf.param
            src = p.detach().to(device=self.device, dtype=torch.float32).reshape(inf.rows, inf.row_numel)
            r0 = self.rank * inf.piece_rows
            r1 = min(inf.rows, r0 + inf.piece_rows)
            if r1 > r0:
                self.master[inf.shard_off: inf.shard_off + (r1 - r0) * inf.row_numel].copy_(src[r0:r1].reshape(-1))
            view = self.flat_param[inf.flat_off: inf.flat_off + p.numel()].view(inf.shape)
            view.copy_(src.view(inf.shape))
            p.data = view
            p.main_grad = self.flat_grad[inf.flat_off: inf.flat_off + p.numel()].view(inf.shape)
            p._main_grad_filled = False
            p._shard_group = self
            p._shard_info = inf

    def _build_tables(self) -> None:
        W, me = self.world, self.rank
        chunk = 1 << 16  # elements per unflagged copy task (128 KB)
        first_tasks: list[tuple[int, int, int, int]] = []
        rest_tasks: list[tuple[int, int, int, int]] = []
        small_tasks: list[tuple[int, int, int, int]] = []
        first_ids = {id(inf) for inf in self.first_gemm_infos}
        # flags cover the rows of the fused first-GEMM operand (its parameters are adjacent)
        self.flag_rows = FLAG_ROWS
        fused_rows = 0
        fused_ok = len(self.first_gemm_infos) > 0
        k = self.first_gemm_infos[0].row_numel if fused_ok else 0
        base = self.first_gemm_infos[0].flat_off if fused_ok else 0
        for inf in self.first_gemm_infos:
            if inf.row_numel != k or inf.flat_off != base + fused_rows * k or inf.rows % W != 0:
                fused_ok = False
            fused_rows += inf.piece_rows * W
        if fused_ok:
            import math as _m

            g = 0
            for inf in self.first_gemm_infos:
                g = _m.gcd(g, inf.piece_rows)
            self.flag_rows = _m.gcd(g, FLAG_ROWS) if g else FLAG_ROWS
            if self.flag_rows < 8:
                fused_ok = False
        self.fused_first = fused_ok and W > 1
        self.fused_rows, self.fused_k, self.fused_base = fused_rows, k, base
        n_flags = max(1, fused_rows // self.flag_rows) if fused_ok else 1
        self.flags = torch.zeros(n_flags, dtype=torch.int32, device=self.device)
        self.local_flag_mask = torch.zeros(n_flags, dtype=torch.bool, device=self.device)
        for step in range(1, W):
            peer = (me + step) % W   # pull order: next rank first, matching the GEMM's tile rotation
            for inf in self.infos:
                poff = inf.flat_off + peer * inf.piece_numel
                n = inf.piece_numel
                # rows past the real end of an unevenly divided parameter are padding
                real = max(0, min(inf.rows, (peer + 1) * inf.piece_rows) - peer * inf.piece_rows) * inf.row_numel
                n = real
                if n == 0:
                    continue
                if len(inf.shape) <= 1 and id(inf) not in first_ids:
                    small_tasks.append((poff, n, peer, -1))
                elif id(inf) in first_ids and self.fused_first:
                    row0 = (poff - base) // k
                    nrows = n // k
                    for r in range(0, nrows, self.flag_rows):
                        first_tasks.append((poff + r * k, self.flag_rows * k, peer, (row0 + r) // self.flag_rows))
                else:
                    for c in range(0, n, chunk):
                        rest_tasks.append((poff + c, min(chunk, n - c), peer, -1))
        if fused_ok:
            for inf in self.first_gemm_infos:
                row0 = (inf.flat_off + me * inf.piece_numel - base) // k
                f0, f1 = row0 // self.flag_rows, (row0 + inf.piece_rows) // self.flag_rows
                self.local_flag_mask[f0:f1] = True
        self.first_tasks = symm.tasks_to_device(first_tasks, self.device) if first_tasks else None
        self.n_first_tasks = len(first_tasks)
        self.rest_tasks = symm.tasks_to_device(rest_tasks, self.device) if rest_tasks else None
        self.n_rest_tasks = len(rest_tasks)
        self.small_tasks = symm.tasks_to_device(small_tasks, self.device) if small_tasks else None
        self.n_small_tasks = len(small_tasks)
        if not self.fused_first and first_tasks == [] and W > 1:
            pass
        self.epoch = 0
        self._segments_dev: torch.Tensor | None = None

    def segments(self) -> torch.Tensor:
        """Device table of this rank's owned slices with their optimizer hyper-parameters."""
        if self._segments_dev is None:
            segs = []
            for inf in self.infos:
                r0 = self.rank * inf.piece_rows
                real = max(0, min(inf.rows, r0 + inf.piece_rows) - r0) * inf.row_numel
                if real > 0:
                    segs.append((inf.flat_off + self.rank * inf.piece_numel, inf.shard_off, real, inf.weight_decay,
                                 inf.lr_scale))
            self._segments_dev = symm.segments_to_device(segs, self.device)
            self._n_segments = len(segs)
        return self._segments_dev

    def set_hyper(self, param: nn.Parameter, weight_decay: float, lr_scale: float = 1.0) -> None:
        inf = param._shard_info
        inf.weight_decay, inf.lr_scale = float(weight_decay), float(lr_scale)
        self._segments_dev = None

    # ---------------------------------------------------------------- all-gather
    def pull(self, which: str, n_ctas: int = 24) -> None:
        """Launch the P2P pull of ``which`` in {"all", "rest", "small", "first"} on the current stream."""
        if self.world == 1:
            return
        l = _lib.lib()
        sets = {"rest": [(self.rest_tasks, self.n_rest_tasks)], "small": [(self.small_tasks, self.n_small_tasks)],
                "first": [(self.first_tasks, self.n_first_tasks)]}
        sets["all"] = sets["small"] + sets["first"] + sets["rest"]
        for tasks, n in sets[which]:
            if tasks is None or n == 0:
                continue
            rc = l.ob_pull(_lib.ptr(tasks), n, self.param_buf.peers.c, self.world, _lib.ptr(self.flat_param),
                           _lib.ptr(self.flags), self.epoch, n_ctas, _lib.stream())
            _lib.check(rc, "ob_pull")

    def begin_epoch(self) -> None:
        """New gather generation: flags of locally owned rows are valid at once."""
        self.epoch += 1
        if self.fused_first:
            self.flags.masked_fill_(self.local_flag_mask, self.epoch)

    def fused_weight(self) -> torch.Tensor:
        return self.flat_param[self.fused_base: self.fused_base + self.fused_rows * self.fused_k].view(self.fused_rows,
                                                                                                       self.fused_k)

    # ---------------------------------------------------------------- reduce-scatter + update
    def zero_grad(self) -> None:
        for inf in self.infos:
            inf.param._main_grad_filled = False
            inf.param.grad = None
        self.grads_reduced = False
        self.updated_in_backward = False

    def fold_autograd_grads(self) -> None:
        """Add gradients that autograd produced as ``.grad`` (norm weights, biases, ...) into the flat buffer."""
        for inf in self.infos:
            p = inf.param
            if p.grad is not None:
                if p._main_grad_filled:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                else:
                    p.main_grad.copy_(p.grad)
                    p._main_grad_filled = True
                p.grad = None
            elif not p._main_grad_filled:
                p.main_grad.zero_()
                p._main_grad_filled = True

    def ensure_state(self, need_grad_shard: bool = False) -> None:
        if self.exp_avg is None:
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
        if need_grad_shard and self.grad_shard is None:
            self.grad_shard = torch.zeros_like(self.master)

    def rs_adamw(self, mode: int, hp: dict, step: int, grad_scale: float, max_norm: float = 0.0,
                 sumsq: torch.Tensor | None = None, scratch: torch.Tensor | None = None, n_ctas: int = 0) -> None:
        segs = self.segments()
        self.ensure_state(need_grad_shard=mode != 0)
        b1, b2 = hp["betas"]
        bc1 = 1.0 - b1 ** step
        bc2 = 1.0 - b2 ** step
        n_ctas = n_ctas or 888
        rc = _lib.lib().ob_rs_adamw(mode, _lib.ptr(segs), self._n_segments, self.grad_buf.peers.c, self.world,
                                    _lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq),
                                    _lib.ptr(self.grad_shard), _lib.ptr(self.flat_param), float(hp["lr"]), float(b1),
                                    float(b2), float(hp["eps"]), bc1, bc2, float(grad_scale), float(max_norm),
                                    _lib.ptr(sumsq) if mode == 2 else None, _lib.ptr(scratch),
                                    _lib.ptr(sumsq) if mode == 1 else None, n_ctas,
                                    _lib.ptr(_lib.status_word(self.device)), _lib.stream())
        _lib.check(rc, "ob_rs_adamw")

    # ---------------------------------------------------------------- state dict helpers
    def local_shard(self, inf: ParamInfo, buf: torch.Tensor) -> torch.Tensor:
        r0 = self.rank * inf.piece_rows
        real_rows = max(0, min(inf.rows, r0 + inf.piece_rows) - r0)
        t = buf[inf.shard_off: inf.shard_off + real_rows * inf.row_numel]
        return t.view(real_rows, *inf.shape[1:]) if len(inf.shape) > 0 else t.view(())

    def refresh_lp_from_master(self) -> None:
        """bf16 rows of this rank <- fp32 master (after an external optimizer or a checkpoint load)."""
        for inf in self.infos:
            r0 = self.rank * inf.piece_rows
            real = max(0, min(inf.rows, r0 + inf.piece_rows) - r0) * inf.row_numel
            if real:
                o = inf.flat_off + self.rank * inf.piece_numel
                self.flat_param[o: o + real].copy_(self.master[inf.shard_off: inf.shard_off + real])
        from ..ops import fp8 as fp8_ops

        fp8_ops.weights_changed()


@dataclass
class FSDPConfig:
    reshard_after_forward: bool = False
    fuse_optimizer_in_backward: bool = True
    copy_ctas: int = 16          # CTAs that pull weights inside the fused all-gather GEMM
    pull_ctas: int = 24          # CTAs of a stand-alone pull
    sync_grad_accum: bool = False


class ShardingEngine:
    """Owns the groups of one model, the side stream and the step protocol."""

    def __init__(self, model: nn.Module, group: Any | None, device: torch.device, units: list[nn.Module],
                 config: FSDPConfig | None = None):
        self.model = model
        self.device = device
        self.cfg = config or FSDPConfig()
        self.heap = symm.SymmetricHeap(group, device)
        self.world, self.rank = self.heap.world, self.heap.rank
        self.pg = group
        self.groups: list[ShardGroup] = []
        self.unit_groups: dict[nn.Module, ShardGroup] = {}
        claimed: set[int] = set()
        for i, unit in enumerate(units):
            named = [(n, p) for n, p in unit.named_parameters() if id(p) not in claimed]
            for _, p in named:
                claimed.add(id(p))
            first = _first_gemm_params(unit)
            g = ShardGroup(f"unit{i}", named, self.heap, device, first)
            self.groups.append(g)
            self.unit_groups[unit] = g
        root_named = [(n, p) for n, p in model.named_parameters() if id(p) not in claimed]
        self.root = ShardGroup("root", root_named, self.heap, device, None)
        self.groups.append(self.root)
        for g in self.groups:
            g.engine = self
        self.barrier = symm.DeviceBarrier(self.heap)
        self.comm_stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self.require_grad_sync = True
        # hybrid sharding: gradients are additionally summed over this group of replicas (one rank per
        # replica holding the same shard) before the update; set by the fully_shard transform
        self.replicate_group: Any | None = None
        self.replicate_world = 1
        self.optimizer: "ShardedAdamW | None" = None
        self._callback_queued = False
        self._step_open = False
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        self.sq_scratch = torch.zeros(1024, dtype=torch.float32, device=device)
        self._install_hooks(units)
        if self.world > 1:
            self._initial_sync()

    # ---------------------------------------------------------------- setup
    def _initial_sync(self) -> None:
        """Make every rank's bf16 parameters equal to the owners' values."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.pg)
        for g in self.groups:
            g.refresh_lp_from_master()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.pg)
        for g in self.groups:
            g.begin_epoch()
            saved = g.fused_first
            g.pull("all", self.cfg.pull_ctas)
            g.gathered = True
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.pg)

    def _install_hooks(self, units: list[nn.Module]) -> None:
        for idx, unit in enumerate(units):
            unit.register_forward_pre_hook(self._make_pre_forward(idx))
            unit.register_full_backward_hook(self._make_post_backward(idx))
        self.model.register_forward_pre_hook(self._root_pre_forward)

    # ---------------------------------------------------------------- forward side
    def _root_pre_forward(self, module: nn.Module, args: Any) -> None:
        if self.world == 1 or all(g.gathered for g in self.groups):
            return
        # parameters were updated by the owners: order the update before any peer read
        self.barrier()
        for g in self.groups:
            if not g.gathered:
                g.begin_epoch()
                g.pull("small", 4)
        if not self.root.gathered:
            self.root.pull("rest", self.cfg.pull_ctas * 2)
            self.root.pull("first", self.cfg.pull_ctas)
            self.root.gathered = True
        # first block: nothing was prefetched yet, pull its non-fused part now (side stream)
        units = list(self.unit_groups.values())
        if units and not units[0].gathered:
            self._prefetch_rest(units[0])

    def _prefetch_rest(self, g: ShardGroup) -> None:
        if g.n_rest_tasks == 0 and (g.fused_first or g.n_first_tasks == 0):
            g.rest_event = None
            return
        cs = self.comm_stream
        cs.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cs):
            g.pull("rest", self.cfg.pull_ctas)
            if not g.fused_first:
                g.pull("first", self.cfg.pull_ctas)
            ev = torch.cuda.Event()
            ev.record(cs)
        g.rest_event = ev

    def _make_pre_forward(self, idx: int):
        def hook(module: nn.Module, args: Any) -> None:
            if self.world == 1:
                return
            g = self.groups[idx]
            if g.gathered:
                return
            if g.rest_event is not None:
                torch.cuda.current_stream().wait_event(g.rest_event)
                g.rest_event = None
            if g.fused_first:
                job = AGJob(g, self.cfg.copy_ctas)
                for inf in g.first_gemm_infos:
                    inf.param._ag_pending = job
            g.gathered = True
            if idx + 1 < len(self.groups) - 1 and not self.groups[idx + 1].gathered:
                self._prefetch_rest(self.groups[idx + 1])

        return hook

    # ---------------------------------------------------------------- backward side
    def _make_post_backward(self, idx: int):
        def hook(module: nn.Module, grad_input: Any, grad_output: Any) -> None:
            self._queue_final_callback()
            if self.require_grad_sync:
                self._reduce_group(self.groups[idx])

        return hook

    def _queue_final_callback(self) -> None:
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._final_callback)

    def _final_callback(self) -> None:
        self._callback_queued = False
        if self.require_grad_sync:
            for g in self.groups:
                if not g.grads_reduced:
                    self._reduce_group(g)
            if self.comm_stream is not None:
                torch.cuda.current_stream().wait_stream(self.comm_stream)

    def finish_backward(self) -> None:
        """Call after ``backward()`` when no unit hook ran (e.g. models without units)."""
        self._final_callback()

    def _reduce_group(self, g: ShardGroup) -> None:
        if g.grads_reduced:
            return
        g.fold_autograd_grads()
        g.grads_reduced = True
        opt = self.optimizer
        fused = (opt is not None and self.cfg.fuse_optimizer_in_backward and opt.max_norm <= 0.0
                 and self.replicate_group is None)
        run_on_side = self.comm_stream is not None
        stream = self.comm_stream if run_on_side else torch.cuda.current_stream()
        if run_on_side:
            stream.wait_stream(torch.cuda.current_stream())
        ctx = torch.cuda.stream(stream) if run_on_side else _nullctx()
        with ctx:
            self.barrier()
            if fused:
                g.rs_adamw(0, opt.hyper(), opt.step_count + 1, opt.grad_scale(self.world))
                g.updated_in_backward = True
                g.gathered = self.world == 1
            else:
                hp = opt.hyper() if opt is not None else dict(lr=0.0, betas=(0.9, 0.999), eps=1e-8)
                g.rs_adamw(1, hp, 1, 1.0, sumsq=self.sumsq, scratch=self.sq_scratch, n_ctas=888)

    # ---------------------------------------------------------------- accumulation / step protocol
    def set_requires_gradient_sync(self, flag: bool) -> None:
        self.require_grad_sync = flag

    def zero_grad(self) -> None:
        for g in self.groups:
            g.zero_grad()
        self.sumsq.zero_()

    def all_params_gathered(self) -> bool:
        return all(g.gathered for g in self.groups)

    def gather_all(self) -> None:
        """Blocking gather of every group (evaluation / checkpoint paths)."""
        if self.world == 1:
            return
        if self.all_params_gathered():
            return
        self.barrier()
        for g in self.groups:
            if not g.gathered:
                g.begin_epoch()
                g.pull("all", self.cfg.pull_ctas)
                g.gathered = True
                g.rest_event = None

    def named_sharded_state(self) -> Iterable[tuple[str, ShardGroup, ParamInfo]]:
        names = {id(p): n for n, p in self.model.named_parameters()}
        for g in self.groups:
            for inf in g.infos:
                yield names.get(id(inf.param), inf.name), g, inf


class AGJob:
    """Pending fused all-gather of a group's first-GEMM weight (consumed by ``ops.linear``)."""

    def __init__(self, group: ShardGroup, copy_ctas: int):
        self.group = group
        self.copy_ctas = copy_ctas
        self.done = False

    def run(self, x2: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        g = self.group
        M, K = x2.shape
        N = g.fused_rows
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x2.device)
        w = g.fused_weight()
        tiles_n = (N + 255) // 256
        # start with the n-tile that holds this rank's first locally owned row
        first_local = (g.first_gemm_infos[0].flat_off + g.rank * g.first_gemm_infos[0].piece_numel - g.fused_base) // g.fused_k
        shift = (first_local // 256) % max(tiles_n, 1)
        rc = _lib.lib().ob_gemm_ag_bf16(_lib.ptr(x2), x2.stride(0), _lib.ptr(w), w.stride(0), _lib.ptr(out),
                                        out.stride(0), M, N, K, _lib.ptr(bias), _lib.ptr(g.first_tasks), g.n_first_tasks,
                                        g.param_buf.peers.c, g.world, _lib.ptr(g.flat_param), _lib.ptr(g.flags),
                                        g.flag_rows, g.epoch, 0, shift, self.copy_ctas,
                                        _lib.ptr(_lib.status_word(x2.device)), _lib.stream())
        _lib.check(rc, "ob_gemm_ag_bf16")
        self.done = True
        for inf in g.first_gemm_infos:
            inf.param._ag_pending = None
        return out

    def gather_only(self, pull_ctas: int = 24) -> None:
        """Complete the gather without the fused GEMM (for consumers that run another kernel on the weight)."""
        if not self.done:
            self.group.pull("first", pull_ctas)
            self.done = True
            for inf in self.group.first_gemm_infos:
                inf.param._ag_pending = None


class _nullctx:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


def _first_gemm_params(unit: nn.Module) -> list[nn.Parameter]:
    """The weights of the first GEMM a transformer block runs (its fused QKV projection)."""
    attn = getattr(unit, "attn", None)
    if attn is not None and all(hasattr(attn, n) for n in ("wq", "wk", "wv")):
        return [attn.wq.weight, attn.wk.weight, attn.wv.weight]
    return []


class ShardedAdamW(torch.optim.Optimizer):
    """AdamW whose state lives in the engine's fp32 shards.

    With ``fuse_optimizer_in_backward`` and no gradient clipping the update of a group has already
    run inside its reduce-scatter kernel when ``step()`` is called; otherwise ``step()`` launches the
    update kernels (with the clip factor computed on the device from the squared norms that the
    reduce kernels accumulated). Hyper-parameters are read at launch time from ``param_groups``,
    so LR schedulers work unchanged.
    """

    def __init__(self, params: Any, engine: ShardingEngine, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, max_norm: float = 0.0, **_: Any):
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        plain = []
        for g in (params if isinstance(params, (list, tuple)) else [params]):
            if isinstance(g, dict):
                gg = dict(g)
                gg["params"] = [p[1] if isinstance(p, tuple) else p for p in gg["params"]]
                plain.append(gg)
            else:
                plain.append(g[1] if isinstance(g, tuple) else g)
        super().__init__(plain, defaults)
        self.engine = engine
        self.max_norm = float(max_norm)
        self.step_count = 0
        engine.optimizer = self
        base_lr = self.param_groups[0]["lr"]
        for pg in self.param_groups:
            for p in pg["params"]:
                sg = getattr(p, "_shard_group", None)
                if sg is None:
                    raise ValueError("ShardedAdamW only takes parameters managed by the sharding engine")
                sg.set_hyper(p, pg["weight_decay"], pg["lr"] / base_lr if base_lr else 1.0)

    def hyper(self) -> dict:
        pg = self.param_groups[0]
        return dict(lr=pg["lr"], betas=pg["betas"], eps=pg["eps"])

    def grad_scale(self, world: int) -> float:
        return 1.0 / (world * max(int(self.engine.replicate_world), 1))

    def set_max_norm(self, max_norm: float | None) -> None:
        self.max_norm = float(max_norm or 0.0)

    @torch.no_grad()
    def step(self, closure=None):
        eng = self.engine
        for g in eng.groups:
            if not g.grads_reduced:
                eng._reduce_group(g)
        if eng.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(eng.comm_stream)
        pending = [g for g in eng.groups if not g.updated_in_backward]
        if pending:
            if eng.replicate_group is not None:
                # sum the reduced fp32 shards over the replicas, then rebuild the squared norm from the sums
                eng.sumsq.zero_()
                for g in pending:
                    dist.all_reduce(g.grad_shard, group=eng.replicate_group)
                    eng.sumsq += g.grad_shard.pow(2).sum()
            if eng.world > 1:
                dist.all_reduce(eng.sumsq, group=eng.pg)
            for g in pending:
                g.rs_adamw(2, self.hyper(), self.step_count + 1, self.grad_scale(eng.world), self.max_norm,
                           sumsq=eng.sumsq if self.max_norm > 0 else None)
                g.gathered = eng.world == 1
        self.step_count += 1
        # the update kernels write parameters through raw pointers (no autograd version bump): tell the caches
        # of derived weight forms (quantised copies) that every parameter changed
        from ..ops import fp8 as fp8_ops

        fp8_ops.weights_changed()
        return None

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last two-phase step (after averaging over ranks)."""
        return self.engine.sumsq.sqrt() * self.grad_scale(self.engine.world)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.engine.zero_grad()

    def state_dict(self) -> dict:
        sd = {"step": self.step_count, "param_groups": [{k: v for k, v in pg.items() if k != "params"} for pg in self.param_groups]}
        return sd

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        for pg, saved in zip(self.param_groups, sd.get("param_groups", [])):
            pg.update({k: v for k, v in saved.items() if k != "params"})


def fully_shard_model(model: nn.Module, group: Any | None, device: torch.device, config: FSDPConfig | None = None,
                      **fsdp_kwargs: Any) -> ShardingEngine:
    """Shard ``model`` in place: one group per unit returned by ``model.fully_shard()`` plus a root group."""
    units = []
    if hasattr(model, "fully_shard"):
        units = list(model.fully_shard(**fsdp_kwargs) or [])
    model.to(device)
    engine = ShardingEngine(model, group, device, units, config)
    model._sharding_engine = engine
    return engine
