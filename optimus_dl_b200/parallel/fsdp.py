"""Fully-sharded data parallelism built on symmetric shard buffers and this package's own kernels.

Semantics follow FSDP2 as the reference uses it (optimus_dl/modules/model_transforms/
distributed.py:187-332; per-model grouping in optimus_dl/modules/model/gpt2.py:325-338):
one parameter group per transformer block plus a root group (embeddings, final norm, head);
every parameter is sharded along dim 0 across the shard group; parameters are computed in bf16
while each rank keeps fp32 master weights and optimizer state for its shard only; gradients are
reduced and accumulated in fp32 and averaged over the data-parallel ranks;
``reshard_after_forward`` and ``shard_every_ith_layer`` choose which blocks give their gathered
parameters back after use.

What differs is the mechanism, which is built for NVLink peer access instead of NCCL:

* Persistent per group and rank: a *symmetric* bf16 buffer with this rank's rows of every
  parameter (``shard_param``) and the fp32 master / moment (/ gradient) shards.
* Gathered parameters live in a *slot*: a local bf16 buffer in the parameter-major flat layout
  (every parameter contiguous and complete, so sibling projections can be fused into one GEMM by
  viewing adjacent parameters as one matrix, ``ops/linear.py``). A resident group owns its slot
  (gathered once per step); resharded groups share a small pool (block ``i`` always uses pool
  slot ``i % pool``, so tensors that autograd saved in the forward see the same memory when the
  block is gathered again for its backward). all-gather = peers' shard rows *pulled* straight
  into the slot (``ob_pull``); for a block the rows of the fused QKV weight are pulled by copy
  CTAs inside the QKV GEMM launch itself, which waits per row group (``ob_gemm_ag_bf16``), and
  the rest of the block is prefetched one block ahead on a side stream.
* Gradients of a block are written into one of three symmetric bf16 *gradient slots* and reduced
  as soon as the block's backward is done: the owner pulls its rows from every peer's slot, adds
  them in a fixed rank order in fp32 and either applies AdamW to its fp32 shard in the same kernel
  (writing the new bf16 values into ``shard_param``) or accumulates into its fp32 gradient shard
  (micro-batches before the last one, gradient clipping, replicas) for the update kernel that
  ``ShardedAdamW.step`` launches (``ob_rs_adamw``). No rank ever holds a full-size gradient buffer.
* Cross-GPU ordering uses a bounded flag barrier (``parallel/symm.DeviceBarrier``). A wait that
  runs out sets the device status word; the update kernels do nothing while it is set, and
  ``ShardedAdamW.step`` reads the word once per step (a copy to pinned memory that is checked at the
  next step, at ``verify()`` and before a checkpoint), so a timed-out step raises instead of
  committing half-reduced gradients.

Per-rank memory for P parameters over W ranks (bf16 compute, fp32 state), besides activations:
resident mode ``2P`` (slots) ``+ 2P/W`` (shard) ``+ 12P/W`` (master, moments) ``+ 4P/W`` (gradient shard,
only when the update is not fused) ``+ 3 x 2 x (largest block)`` (gradient slots) ``+ 2 x root`` (root gradient);
resharded mode replaces the first term by ``pool x 2 x (largest block) + 2 x root``.

A world of one runs the same code: the shard is the whole parameter, the slot is the shard buffer
itself and nothing is pulled, which is how the single-GPU benchmark exercises the identical kernels.
"""

from __future__ import annotations

import logging
import math
from dataclasses import dataclass
from typing import Any, Iterable

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _lib
from ..ops import gemm as gemm_ops
from ..ops import optim as optim_ops
from . import symm

logger = logging.getLogger(__name__)

ALIGN = 8          # elements: 16 bytes of bf16, the vector width of the copy / update kernels
FLAG_ROWS = 128    # rows of the gathered QKV weight guarded by one readiness flag
GRAD_SLOTS = 3     # symmetric gradient buffers shared by the block groups


@dataclass
class ParamInfo:
    name: str
    param: nn.Parameter
    shape: tuple
    rows: int
    row_numel: int
    piece_rows: int        # rows owned by each rank (dim 0 padded up to a multiple of world)
    flat_off: int          # element offset of the parameter in the flat (gathered / gradient) layout
    shard_off: int = 0     # element offset of this rank's piece in the shard layout (bf16 shard and fp32 state)
    weight_decay: float = 0.0
    lr_scale: float = 1.0

    @property
    def piece_numel(self) -> int:
        return self.piece_rows * self.row_numel


class GatherSlot:
    """Local bf16 buffer that holds the gathered parameters of one group at a time."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor
        self.owner: "ShardGroup | None" = None
        self.ready: torch.cuda.Event | None = None      # recorded on the stream that ran the pull
        self.first_pending = False                       # rows of the fused first GEMM still to be pulled by that GEMM


class GradSlot:
    """Symmetric bf16 buffer the wgrad kernels of one group write and every rank's reduce kernel reads."""

    def __init__(self, buf: symm.SymmetricBuffer):
        self.buf = buf
        self.tensor = buf.tensor


class ShardGroup:
    """One sharding unit: this rank's bf16 / fp32 shards, the flat layout of the gathered parameters and the copy
    and segment tables the kernels use."""

    def __init__(self, name: str, named_params: list[tuple[str, nn.Parameter]], heap: symm.SymmetricHeap,
                 device: torch.device, first_gemm_params: list[nn.Parameter] | None = None):
        self.name = name
        self.heap = heap
        self.device = device
        self.world, self.rank = heap.world, heap.rank
        W = self.world
        self.infos: list[ParamInfo] = []
        off = soff = 0
        # the parameters consumed by the group's first GEMM go first and back to back
        first_ids = [id(p) for p in (first_gemm_params or [])]
        ordered = sorted(named_params, key=lambda np_: (first_ids.index(id(np_[1])) if id(np_[1]) in first_ids else len(first_ids)))
        for pname, p in ordered:
            shape = tuple(p.shape)
            rows = shape[0] if len(shape) > 0 else 1
            row_numel = max(1, p.numel() // max(rows, 1))
            piece_rows = math.ceil(rows / W)
            off = (off + ALIGN - 1) // ALIGN * ALIGN
            soff = (soff + ALIGN - 1) // ALIGN * ALIGN
            self.infos.append(ParamInfo(pname, p, shape, rows, row_numel, piece_rows, off, soff))
            off += piece_rows * W * row_numel
            soff += piece_rows * row_numel
        self.flat_numel = (off + ALIGN - 1) // ALIGN * ALIGN
        self.shard_numel = (soff + ALIGN - 1) // ALIGN * ALIGN
        self.shard_buf = heap.empty(self.shard_numel, torch.bfloat16, zero=True)
        self.shard_param = self.shard_buf.tensor
        self.master = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        self.exp_avg: torch.Tensor | None = None
        self.exp_avg_sq: torch.Tensor | None = None
        self.grad_shard: torch.Tensor | None = None
        self.grad_shard_filled = False
        self.first_gemm_infos = [inf for inf in self.infos if id(inf.param) in first_ids]
        self.slot: GatherSlot | None = None
        self.grad_slot: GradSlot | None = None
        self.pooled = False
        self.index = -1
        self.reduce_event: torch.cuda.Event | None = None
        self.backward_prepared = False
        self.grads_reduced = False
        self.updated_in_backward = False
        self.epoch = 0
        self._segments_dev: torch.Tensor | None = None
        self._n_segments = 0
        self._take_initial_values()

    # ---------------------------------------------------------------- construction
    def real_piece(self, inf: ParamInfo, rank: int) -> int:
        """Elements of ``inf`` that rank ``rank`` really owns (rows past the end of an unevenly divided parameter
        are padding)."""
        r0 = rank * inf.piece_rows
        return max(0, min(inf.rows, r0 + inf.piece_rows) - r0) * inf.row_numel

    def _take_initial_values(self) -> None:
        """fp32 masters and bf16 shard rows of this rank from the parameters' current values."""
        for inf in self.infos:
            p = inf.param
            src = p.detach().to(device=self.device, dtype=torch.float32).reshape(inf.rows, inf.row_numel)
            n = self.real_piece(inf, self.rank)
            if n:
                r0 = self.rank * inf.piece_rows
                piece = src[r0: r0 + n // inf.row_numel].reshape(-1)
                self.master[inf.shard_off: inf.shard_off + n].copy_(piece)
                self.shard_param[inf.shard_off: inf.shard_off + n].copy_(piece)
            p._shard_group = self
            p._shard_info = inf
            p._main_grad_filled = False

    def bind(self, slot: GatherSlot, grad_slot: GradSlot, pooled: bool) -> None:
        """Point the parameters at their place in ``slot`` (data) and ``grad_slot`` (``main_grad``). The views are
        fixed for the life of the engine; for pooled groups they alias the other groups of the same pool slot."""
        self.slot, self.grad_slot, self.pooled = slot, grad_slot, pooled
        for inf in self.infos:
            p = inf.param
            n = p.numel()
            old = p.data
            p.data = slot.tensor[inf.flat_off: inf.flat_off + n].view(inf.shape)
            p.main_grad = grad_slot.tensor[inf.flat_off: inf.flat_off + n].view(inf.shape)
            del old
        self._build_tables()

    def _build_tables(self) -> None:
        W, me = self.world, self.rank
        chunk = 1 << 16  # elements per unflagged copy task (128 KB)
        first_tasks: list[tuple] = []
        rest_tasks: list[tuple] = []
        small_tasks: list[tuple] = []
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
            g = 0
            for inf in self.first_gemm_infos:
                g = math.gcd(g, inf.piece_rows)
            self.flag_rows = math.gcd(g, FLAG_ROWS) if g else FLAG_ROWS
            if self.flag_rows < 8:
                fused_ok = False
        self.fused_first = fused_ok and W > 1
        self.fused_rows, self.fused_k, self.fused_base = fused_rows, k, base
        n_flags = max(1, fused_rows // self.flag_rows) if fused_ok else 1
        self.flags = torch.zeros(n_flags, dtype=torch.int32, device=self.device)
        if W > 1:
            for step in range(W):
                peer = (me + step) % W   # pull order: own rows, then the next rank's, matching the GEMM's tile rotation
                for inf in self.infos:
                    dst = inf.flat_off + peer * inf.piece_numel
                    src = inf.shard_off
                    n = self.real_piece(inf, peer)
                    if n == 0:
                        continue
                    if len(inf.shape) <= 1 and id(inf) not in first_ids:
                        small_tasks.append((dst, n, peer, -1, src))
                    elif id(inf) in first_ids and self.fused_first:
                        row0 = (dst - base) // k
                        for r in range(0, n // k, self.flag_rows):
                            first_tasks.append((dst + r * k, self.flag_rows * k, peer, (row0 + r) // self.flag_rows, src + r * k))
                    else:
                        for c in range(0, n, chunk):
                            rest_tasks.append((dst + c, min(chunk, n - c), peer, -1, src + c))
        self.first_tasks = symm.tasks_to_device(first_tasks, self.device) if first_tasks else None
        self.n_first_tasks = len(first_tasks)
        self.rest_tasks = symm.tasks_to_device(rest_tasks, self.device) if rest_tasks else None
        self.n_rest_tasks = len(rest_tasks)
        self.small_tasks = symm.tasks_to_device(small_tasks, self.device) if small_tasks else None
        self.n_small_tasks = len(small_tasks)

    def segments(self) -> torch.Tensor:
        """Device table of this rank's owned slices with their optimizer hyper-parameters."""
        if self._segments_dev is None:
            segs = []
            for inf in self.infos:
                real = self.real_piece(inf, self.rank)
                if real > 0:
                    segs.append((inf.flat_off + self.rank * inf.piece_numel, inf.shard_off, inf.shard_off, real,
                                 inf.weight_decay, inf.lr_scale))
            self._segments_dev = symm.segments_to_device(segs, self.device)
            self._n_segments = len(segs)
        return self._segments_dev

    def set_hyper(self, param: nn.Parameter, weight_decay: float, lr_scale: float = 1.0) -> None:
        inf = param._shard_info
        if inf.weight_decay != float(weight_decay) or inf.lr_scale != float(lr_scale):
            inf.weight_decay, inf.lr_scale = float(weight_decay), float(lr_scale)
            self._segments_dev = None

    # ---------------------------------------------------------------- all-gather
    @property
    def gathered(self) -> bool:
        return self.world == 1 or (self.slot is not None and self.slot.owner is self)

    @gathered.setter
    def gathered(self, value: bool) -> None:
        if not value:
            self.invalidate()

    def invalidate(self) -> None:
        """The shard rows changed (optimizer step, checkpoint load): the gathered copy is stale."""
        if self.world > 1 and self.slot is not None and self.slot.owner is self:
            self.slot.owner = None
            self.slot.ready = None
            self.slot.first_pending = False

    def pull(self, which: str, n_ctas: int = 24) -> None:
        """Launch the P2P pull of ``which`` in {"all", "rest", "small", "first"} into the group's slot on the current
        stream."""
        if self.world == 1:
            return
        l = _lib.lib()
        sets = {"rest": [(self.rest_tasks, self.n_rest_tasks)], "small": [(self.small_tasks, self.n_small_tasks)],
                "first": [(self.first_tasks, self.n_first_tasks)]}
        sets["all"] = sets["small"] + sets["first"] + sets["rest"]
        for tasks, n in sets[which]:
            if tasks is None or n == 0:
                continue
            rc = l.ob_pull(_lib.ptr(tasks), n, self.shard_buf.peers.c, self.world, _lib.ptr(self.slot.tensor),
                           _lib.ptr(self.flags), self.epoch, n_ctas, _lib.stream())
            _lib.check(rc, "ob_pull")

    def fused_weight(self) -> torch.Tensor:
        return self.slot.tensor[self.fused_base: self.fused_base + self.fused_rows * self.fused_k].view(self.fused_rows,
                                                                                                        self.fused_k)

    # ---------------------------------------------------------------- reduce-scatter + update
    def zero_grad(self) -> None:
        for inf in self.infos:
            inf.param._main_grad_filled = False
            inf.param.grad = None
        self.grads_reduced = False
        self.updated_in_backward = False
        self.grad_shard_filled = False
        self.backward_prepared = False

    def fold_autograd_grads(self) -> None:
        """Add gradients that autograd produced as ``.grad`` (norm weights, biases, ...) into the gradient slot."""
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
                 sumsq: torch.Tensor | None = None, acc_in: bool = False, n_ctas: int = 0) -> None:
        segs = self.segments()
        self.ensure_state(need_grad_shard=mode != 0 or acc_in)
        b1, b2 = hp["betas"]
        bc1 = 1.0 - b1 ** step
        bc2 = 1.0 - b2 ** step
        n_ctas = n_ctas or 888
        rc = _lib.lib().ob_rs_adamw(mode, _lib.ptr(segs), self._n_segments, self.grad_slot.buf.peers.c, self.world,
                                    _lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq),
                                    _lib.ptr(self.grad_shard), _lib.ptr(self.shard_param), float(hp["lr"]), float(b1),
                                    float(b2), float(hp["eps"]), bc1, bc2, float(grad_scale), float(max_norm),
                                    _lib.ptr(sumsq) if (mode == 2 and sumsq is not None) else None, int(acc_in), n_ctas,
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
        self.shard_param.copy_(self.master)
        self.invalidate()
        from ..ops import fp8 as fp8_ops

        fp8_ops.weights_changed()


@dataclass
class FSDPConfig:
    reshard_after_forward: bool = False
    fuse_optimizer_in_backward: bool = True
    copy_ctas: int = 16          # CTAs that pull weights inside the fused all-gather GEMM
    pull_ctas: int = 24          # CTAs of a stand-alone pull
    sync_grad_accum: bool = False
    param_slots: int = 2         # size of the pool that resharded blocks are gathered into
    shard_every_ith_layer: int = 1   # with reshard_after_forward: only blocks with index % i == 0 are resharded


class ShardingEngine:
    """Owns the groups of one model, the slots, the side stream and the step protocol."""

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
            g = ShardGroup(f"unit{i}", named, self.heap, device, _first_gemm_params(unit))
            g.index = i
            self.groups.append(g)
            self.unit_groups[unit] = g
        root_named = [(n, p) for n, p in model.named_parameters() if id(p) not in claimed]
        self.root = ShardGroup("root", root_named, self.heap, device, None)
        self.root.index = len(self.groups)
        self.groups.append(self.root)
        self._bind_slots()
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
        self._in_backward = False
        self._reduced_since_barrier = False
        self.micro_batch = 0             # micro-batches reduced since the last zero_grad
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        self.status = _lib.DeferredStatus(device)
        self._install_hooks(units)
        if self.world > 1:
            # every rank's shard rows are in place before any peer pulls them; resident groups are gathered right
            # away so that the parameters hold their values before the first forward pass
            self.host_sync()
            if not any(g.pooled for g in self.groups):
                self.gather_all()
                self.host_sync()

    # ---------------------------------------------------------------- setup
    def _bind_slots(self) -> None:
        """Give every group its gathered-parameter slot and gradient slot (see the module docstring)."""
        units = self.groups[:-1]
        W = self.world
        reshard = bool(self.cfg.reshard_after_forward) and W > 1
        ith = max(int(self.cfg.shard_every_ith_layer or 1), 1)
        pooled = [reshard and (g.index % ith == 0) for g in units]
        dev = self.device
        pool: list[GatherSlot] = []
        if any(pooled):
            size = max(g.flat_numel for g, p in zip(units, pooled) if p)
            pool = [GatherSlot(torch.zeros(size, dtype=torch.bfloat16, device=dev))
                    for _ in range(max(2, int(self.cfg.param_slots)))]
        grad_pool: list[GradSlot] = []
        if units:
            gsize = max(g.flat_numel for g in units)
            grad_pool = [GradSlot(self.heap.empty(gsize, torch.bfloat16, zero=True)) for _ in range(min(GRAD_SLOTS, len(units)))]
        n_pooled = 0
        for g, is_pooled in zip(units, pooled):
            if W == 1:
                slot = GatherSlot(g.shard_param)
                slot.owner = g
            elif is_pooled:
                slot = pool[n_pooled % len(pool)]
                n_pooled += 1
            else:
                slot = GatherSlot(torch.zeros(g.flat_numel, dtype=torch.bfloat16, device=dev))
            g.bind(slot, grad_pool[g.index % len(grad_pool)], is_pooled)
        root = self.root
        rslot = GatherSlot(root.shard_param if W == 1 else torch.zeros(root.flat_numel, dtype=torch.bfloat16, device=dev))
        if W == 1:
            rslot.owner = root
        root.bind(rslot, GradSlot(self.heap.empty(root.flat_numel, torch.bfloat16, zero=True)), False)
        self.param_pool, self.grad_pool = pool, grad_pool

    def _install_hooks(self, units: list[nn.Module]) -> None:
        for idx, unit in enumerate(units):
            unit.register_forward_pre_hook(self._make_pre_forward(idx))
            unit.register_full_backward_pre_hook(self._make_pre_backward(idx))
            unit.register_full_backward_hook(self._make_post_backward(idx))
        self.model.register_forward_pre_hook(self._root_pre_forward)

    # ---------------------------------------------------------------- gathering
    def _start_gather(self, g: ShardGroup, *, leave_first: bool) -> None:
        """Queue the pull of ``g`` into its slot on the side stream (after everything queued so far on the compute
        stream, which includes the previous user of a pooled slot). With ``leave_first`` the rows of the fused
        first GEMM are left to that GEMM's launch."""
        slot = g.slot
        slot.owner = g
        g.epoch += 1
        cs = self.comm_stream
        cs.wait_stream(torch.cuda.current_stream())
        fused = g.fused_first and leave_first
        with torch.cuda.stream(cs):
            g.pull("small", 4)
            g.pull("rest", self.cfg.pull_ctas)
            if not fused:
                g.pull("first", self.cfg.pull_ctas)
            ev = torch.cuda.Event()
            ev.record(cs)
        slot.ready = ev
        slot.first_pending = fused

    def _ensure_gathered(self, g: ShardGroup, *, leave_first: bool) -> None:
        """Make the compute stream see ``g``'s parameters in its slot (gathering now if nobody prefetched them)."""
        if self.world == 1:
            return
        slot = g.slot
        if slot.owner is not g:
            self._start_gather(g, leave_first=leave_first)
        if slot.ready is not None:
            torch.cuda.current_stream().wait_event(slot.ready)
            slot.ready = None
        if slot.first_pending:
            if leave_first:
                job = AGJob(g, self.cfg.copy_ctas)
                for inf in g.first_gemm_infos:
                    inf.param._ag_pending = job
            else:
                g.pull("first", self.cfg.pull_ctas)
            slot.first_pending = False

    def _step_barrier(self) -> None:
        """Once per micro-batch, before the first peer read of the forward: every rank has finished the reduce /
        update kernels of the previous backward (they read this rank's gradient slots and wrote the shard rows)."""
        if self.world > 1 and self._reduced_since_barrier:
            if self.comm_stream is not None:
                torch.cuda.current_stream().wait_stream(self.comm_stream)
            self.barrier()
            self._reduced_since_barrier = False

    # ---------------------------------------------------------------- forward side
    def _root_pre_forward(self, module: nn.Module, args: Any) -> None:
        if self.world == 1:
            return
        self._in_backward = False
        self._step_barrier()
        if not self.root.gathered:
            self.root.slot.owner = self.root
            self.root.epoch += 1
            self.root.pull("all", self.cfg.pull_ctas * 2)
        units = self.groups[:-1]
        if units and not units[0].gathered:
            self._start_gather(units[0], leave_first=True)

    def _make_pre_forward(self, idx: int):
        def hook(module: nn.Module, args: Any) -> None:
            if self.world == 1:
                return
            g = self.groups[idx]
            recompute = self._in_backward      # activation checkpointing re-runs the block inside the backward pass
            self._ensure_gathered(g, leave_first=not recompute)
            if not recompute and idx + 1 < len(self.groups) - 1:
                nxt = self.groups[idx + 1]
                if not nxt.gathered:
                    self._start_gather(nxt, leave_first=True)

        return hook

    # ---------------------------------------------------------------- backward side
    def _prepare_backward(self, g: ShardGroup) -> None:
        """Before the first gradient kernel of ``g`` in a backward pass: its gradient slot is free again. The slot's
        previous user in this pass is the block K = len(grad_pool) positions later; every rank has finished reducing
        that block once this rank has passed the barrier of the NEXT reduce (block index + K - 1), whose completion
        event the compute stream waits for."""
        if g.backward_prepared:
            return
        g.backward_prepared = True
        units = self.groups[:-1]
        K = len(self.grad_pool)
        if g is not self.root and K > 1:
            j = g.index + K - 1
            if j < len(units) and units[j].reduce_event is not None:
                torch.cuda.current_stream().wait_event(units[j].reduce_event)

    def _make_pre_backward(self, idx: int):
        def hook(module: nn.Module, grad_output: Any) -> None:
            self._in_backward = True
            g = self.groups[idx]
            self._prepare_backward(g)
            if self.world > 1:
                self._ensure_gathered(g, leave_first=False)
                if idx > 0:
                    prv = self.groups[idx - 1]
                    if not prv.gathered:
                        self._start_gather(prv, leave_first=False)

        return hook

    def _make_post_backward(self, idx: int):
        def hook(module: nn.Module, grad_input: Any, grad_output: Any) -> None:
            self._queue_final_callback()
            self._reduce_group(self.groups[idx])

        return hook

    def _queue_final_callback(self) -> None:
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._final_callback)

    def _final_callback(self) -> None:
        self._callback_queued = False
        for g in self.groups:
            if not g.grads_reduced:
                self._reduce_group(g)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._in_backward = False
        self.micro_batch += 1
        for g in self.groups:           # ready for the next micro-batch of the same step
            g.grads_reduced = False
            g.backward_prepared = False
            g.reduce_event = None
            for inf in g.infos:
                inf.param._main_grad_filled = False

    def finish_backward(self) -> None:
        """Call after ``backward()`` when no unit hook ran (e.g. models without units)."""
        self._final_callback()

    def _reduce_group(self, g: ShardGroup) -> None:
        """Reduce ``g``'s gradient slot over the ranks: into the fused AdamW update when this is the only or last
        micro-batch of a step without clipping and replicas, into the fp32 gradient shard otherwise."""
        if g.grads_reduced:
            return
        self._prepare_backward(g)
        g.fold_autograd_grads()
        g.grads_reduced = True
        opt = self.optimizer
        last = self.require_grad_sync
        fused = (opt is not None and self.cfg.fuse_optimizer_in_backward and opt.max_norm <= 0.0
                 and self.replicate_group is None and last)
        run_on_side = self.comm_stream is not None
        stream = self.comm_stream if run_on_side else torch.cuda.current_stream()
        if run_on_side:
            stream.wait_stream(torch.cuda.current_stream())
        ctx = torch.cuda.stream(stream) if run_on_side else _nullctx()
        with ctx:
            self.barrier()
            acc = g.grad_shard_filled
            if fused:
                opt.refresh_hyper()
                g.rs_adamw(0, opt.hyper(), opt.step_count + 1, opt.grad_scale(self.world), acc_in=acc)
                g.updated_in_backward = True
                g.invalidate()
            else:
                g.rs_adamw(1, dict(lr=0.0, betas=(0.9, 0.999), eps=1e-8), 1, 1.0, acc_in=acc)
                g.grad_shard_filled = True
            if run_on_side:
                ev = torch.cuda.Event()
                ev.record(stream)
                g.reduce_event = ev
        self._reduced_since_barrier = True

    # ---------------------------------------------------------------- accumulation / step protocol
    def set_requires_gradient_sync(self, flag: bool) -> None:
        """``False`` marks a micro-batch that is not the last of its step. Gradients are still reduced after every
        micro-batch (into the fp32 gradient shards: no rank keeps full-size gradients), so the flag only decides
        whether the reduce may apply the optimizer update at once."""
        self.require_grad_sync = flag

    def zero_grad(self) -> None:
        for g in self.groups:
            g.zero_grad()
        self.micro_batch = 0

    def all_params_gathered(self) -> bool:
        return all(g.gathered for g in self.groups)

    def gather_all(self) -> None:
        """Blocking gather of every resident group (evaluation / generation / checkpoint paths). Resharded groups
        have no slot of their own; they are gathered block by block when a forward pass reaches them."""
        if self.world == 1:
            return
        if any(g.pooled for g in self.groups):
            raise RuntimeError("gather_all() needs resident parameters: this model was sharded with reshard_after_forward, "
                               "run forward passes through the model (its hooks gather block by block) instead")
        if self.all_params_gathered():
            return
        self._step_barrier()
        for g in self.groups:
            if not g.gathered:
                self._ensure_gathered(g, leave_first=False)

    def verify(self) -> None:
        """Synchronously check that no kernel of the steps so far reported a failed wait (call before anything that
        persists state: checkpoints, the end of training)."""
        self.status.event = None
        _lib.check_status(self.device)

    def host_sync(self) -> None:
        """Device synchronisation plus a host-side barrier over the shard group: call after long per-rank host work
        (checkpoint writing, evaluation, the first batch) so that ordinary skew between ranks never gets near the
        kernels' bounded waits."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.pg)

    def memory_bytes(self) -> dict:
        """Bytes of device memory this engine holds on this rank, by purpose."""
        bf, f4 = 2, 4
        slots = {id(g.slot): g.slot.tensor.numel() * bf for g in self.groups if self.world > 1}
        gslots = {id(g.grad_slot): g.grad_slot.tensor.numel() * bf for g in self.groups}
        n_state = sum(2 if g.exp_avg is not None else 0 for g in self.groups)
        return {"gathered_parameter_slots": sum(slots.values()), "gradient_slots": sum(gslots.values()),
                "bf16_shards": sum(g.shard_numel for g in self.groups) * bf,
                "fp32_master": sum(g.shard_numel for g in self.groups) * f4,
                "fp32_moments": sum(g.shard_numel * (2 if g.exp_avg is not None else 0) for g in self.groups) * f4,
                "fp32_grad_shards": sum(g.shard_numel for g in self.groups if g.grad_shard is not None) * f4,
                "_groups_with_moments": n_state // 2}

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
        l = _lib.lib()
        if gemm_ops.USE_2SM and ((M + 255) // 256) * tiles_n >= gemm_ops.PAIR_MIN_TILES - self.copy_ctas // 2:
            # two-SM tiles, copy CTAs in pairs (csrc/gemm_ag.cu: ob_gemm2_ag_bf16)
            rc = l.ob_gemm2_ag_bf16(_lib.ptr(x2), x2.stride(0), _lib.ptr(w), w.stride(0), _lib.ptr(out), out.stride(0),
                                    M, N, K, _lib.ptr(bias), _lib.ptr(g.first_tasks), g.n_first_tasks,
                                    g.shard_buf.peers.c, g.world, _lib.ptr(g.slot.tensor), _lib.ptr(g.flags),
                                    g.flag_rows, g.epoch, shift, self.copy_ctas,
                                    _lib.ptr(_lib.status_word(x2.device)), _lib.stream())
        else:
            rc = l.ob_gemm_ag_bf16(_lib.ptr(x2), x2.stride(0), _lib.ptr(w), w.stride(0), _lib.ptr(out),
                                   out.stride(0), M, N, K, _lib.ptr(bias), _lib.ptr(g.first_tasks), g.n_first_tasks,
                                   g.shard_buf.peers.c, g.world, _lib.ptr(g.slot.tensor), _lib.ptr(g.flags),
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
    run inside its reduce kernel when ``step()`` is called; otherwise ``step()`` launches the
    update kernels (with the clip factor computed on the device from the squared norm of the fp32
    gradient shards). Learning rate, weight decay and the per-group learning-rate ratio are read from
    ``param_groups`` at launch time, so LR schedulers and later changes work unchanged; ``betas`` and
    ``eps`` must be the same in every group (one kernel launch covers a whole sharding group).
    ``step()`` also queues the per-step read of the device status word (see the module docstring).
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
        for pg in self.param_groups:
            for p in pg["params"]:
                if getattr(p, "_shard_group", None) is None:
                    raise ValueError("ShardedAdamW only takes parameters managed by the sharding engine")
        self._hyper_key: tuple | None = None
        self.refresh_hyper()

    def refresh_hyper(self) -> None:
        """Push the param groups' current weight decay and learning-rate ratio into the kernels' segment tables
        (only when something changed) and check that the settings one launch shares are uniform."""
        key = tuple((pg["lr"], pg["weight_decay"], tuple(pg["betas"]), pg["eps"]) for pg in self.param_groups)
        if key == self._hyper_key:
            return
        first = self.param_groups[0]
        for pg in self.param_groups[1:]:
            if tuple(pg["betas"]) != tuple(first["betas"]) or pg["eps"] != first["eps"]:
                raise ValueError("ShardedAdamW: betas and eps must be equal in all parameter groups "
                                 f"(got {pg['betas']}, {pg['eps']} vs {first['betas']}, {first['eps']})")
        base_lr = first["lr"]
        for pg in self.param_groups:
            for p in pg["params"]:
                p._shard_group.set_hyper(p, pg["weight_decay"], pg["lr"] / base_lr if base_lr else 1.0)
        self._hyper_key = key

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
        eng.status.check()              # a failed wait in the previous step: raise before anything else is committed
        self.refresh_hyper()
        for g in eng.groups:
            if not g.grads_reduced and not g.updated_in_backward and not g.grad_shard_filled:
                eng._reduce_group(g)
        if eng.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(eng.comm_stream)
        pending = [g for g in eng.groups if not g.updated_in_backward]
        if pending:
            if eng.replicate_group is not None:
                # sum the reduced fp32 shards over the replicas
                for g in pending:
                    dist.all_reduce(g.grad_shard, group=eng.replicate_group)
            if self.max_norm > 0:
                for i, g in enumerate(pending):
                    optim_ops.sumsq_(g.grad_shard, eng.sumsq, accumulate=i > 0)
                if eng.world > 1:
                    dist.all_reduce(eng.sumsq, group=eng.pg)
            for g in pending:
                g.rs_adamw(2, self.hyper(), self.step_count + 1, self.grad_scale(eng.world), self.max_norm,
                           sumsq=eng.sumsq if self.max_norm > 0 else None)
                g.invalidate()
            eng._reduced_since_barrier = True
        self.step_count += 1
        eng.status.post()
        # the update kernels write parameters through raw pointers (no autograd version bump): tell the caches
        # of derived weight forms (quantised copies) that every parameter changed
        from ..ops import fp8 as fp8_ops

        fp8_ops.weights_changed()
        return None

    def grad_norm(self) -> torch.Tensor:
        """Global gradient norm of the last clipped step (after averaging over ranks)."""
        return self.engine.sumsq.sqrt() * self.grad_scale(self.engine.world)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.engine.zero_grad()

    def state_dict(self) -> dict:
        """Step count, parameter-group scalars and this rank's fp32 shards (``torch.save`` form; distributed
        checkpoints use ``parallel/state.py``, which wraps the same tensors as DTensors)."""
        shards = {}
        for g in self.engine.groups:
            g.ensure_state()
            shards[g.name] = {"master": g.master, "exp_avg": g.exp_avg, "exp_avg_sq": g.exp_avg_sq}
        return {"step": self.step_count, "shards": shards,
                "param_groups": [{k: v for k, v in pg.items() if k != "params"} for pg in self.param_groups]}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step", 0))
        for pg, saved in zip(self.param_groups, sd.get("param_groups", [])):
            pg.update({k: v for k, v in saved.items() if k != "params"})
        for g in self.engine.groups:
            st = sd.get("shards", {}).get(g.name)
            if st is not None:
                g.ensure_state()
                g.master.copy_(st["master"])
                g.exp_avg.copy_(st["exp_avg"])
                g.exp_avg_sq.copy_(st["exp_avg_sq"])
                g.refresh_lp_from_master()
        self._hyper_key = None


def fully_shard_model(model: nn.Module, group: Any | None, device: torch.device, config: FSDPConfig | None = None,
                      **fsdp_kwargs: Any) -> ShardingEngine:
    """Shard ``model`` in place: one group per unit returned by ``model.fully_shard()`` plus a root group."""
    units = []
    if hasattr(model, "fully_shard"):
        units = list(model.fully_shard(**fsdp_kwargs) or [])
    config = config or FSDPConfig()
    ith = getattr(getattr(model, "config", None), "shard_every_ith_layer", None)
    if ith is not None and config.shard_every_ith_layer == 1:
        config.shard_every_ith_layer = max(int(ith), 1)
    model.to(device)
    engine = ShardingEngine(model, group, device, units, config)
    model._sharding_engine = engine
    return engine
