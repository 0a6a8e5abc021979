"""Symmetric peer memory: buffers every rank of a group can address from inside a kernel.

``SymmetricHeap(group)`` allocates tensors at the same offset on every rank and exchanges the
mappings once, so kernels receive an array of peer base pointers and use plain loads / stores
over NVLink (``csrc/comm.cuh``). Allocation and handle exchange use PyTorch's symmetric-memory
allocator (CUDA VMM handles over the process group's store); the data plane — pulls, flags,
barriers, reductions — is this package's own kernels. With a world of one the "peer" list is
just the local pointer, so the same kernels run unchanged on a single GPU.

``DeviceBarrier`` is a stream-ordered cross-GPU barrier on a symmetric flag array whose waits
are bounded: a rank that never arrives makes the others record ``flag wait timed out`` in the
status word instead of hanging (see ``ops/_lib.check_status``).
"""

from __future__ import annotations

import ctypes
import logging
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib

logger = logging.getLogger(__name__)


class PeerArray:
    """A ``void*[world]`` kept alive on the host for ctypes calls."""

    def __init__(self, ptrs: list[int]):
        self.ptrs = list(ptrs)
        self._arr = (ctypes.c_void_p * len(ptrs))(*ptrs)

    @property
    def c(self) -> Any:
        return self._arr


class SymmetricBuffer:
    """One symmetric allocation: the local tensor plus every rank's base pointer."""

    def __init__(self, tensor: torch.Tensor, peer_ptrs: list[int], handle: Any = None):
        self.tensor = tensor
        self.peers = PeerArray(peer_ptrs)
        self.handle = handle

    def offset_peers(self, byte_offset: int) -> PeerArray:
        return PeerArray([p + byte_offset for p in self.peers.ptrs])


class SymmetricHeap:
    def __init__(self, group: Any | None, device: torch.device):
        self.group = group
        self.device = device
        if group is None or not dist.is_initialized():
            self.world, self.rank = 1, 0
        else:
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self._symm = None
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            self._symm = symm_mem
            self._group_name = group.group_name if hasattr(group, "group_name") else dist.group.WORLD.group_name
            try:
                symm_mem.enable_symm_mem_for_group(self._group_name)
            except Exception as e:  # newer torch versions enable lazily
                logger.debug("enable_symm_mem_for_group: %s", e)

    def empty(self, numel: int, dtype: torch.dtype, zero: bool = False) -> SymmetricBuffer:
        numel = max(int(numel), 1)
        if self.world == 1:
            t = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=self.device)
            return SymmetricBuffer(t, [t.data_ptr()])
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        hdl = self._symm.rendezvous(t, self._group_name)
        if zero:
            t.zero_()
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        ptrs[self.rank] = t.data_ptr()
        return SymmetricBuffer(t, ptrs, hdl)


class DeviceBarrier:
    """Bounded cross-GPU barrier (``ob_barrier``) over a symmetric int32 flag array."""

    def __init__(self, heap: SymmetricHeap):
        self.heap = heap
        self.buf = heap.empty(64, torch.int32, zero=True)
        self.epoch = 0
        if heap.world > 1:
            # make the zero-initialisation visible everywhere before the first use
            torch.cuda.synchronize(heap.device)
            dist.barrier(group=heap.group)

    def __call__(self) -> None:
        if self.heap.world == 1:
            return
        self.epoch += 1
        rc = _lib.lib().ob_barrier(self.buf.peers.c, self.heap.rank, self.heap.world, self.epoch,
                                   _lib.ptr(_lib.status_word(self.heap.device)), _lib.stream())
        _lib.check(rc, "ob_barrier")


COPY_TASK_DTYPE = np.dtype([("offset", "<i8"), ("src_offset", "<i8"), ("numel", "<i4"), ("peer", "<i2"), ("pad", "<i2"),
                            ("flag", "<i4"), ("pad2", "<i4")])
SEGMENT_DTYPE = np.dtype([("grad_off", "<i8"), ("param_off", "<i8"), ("shard_off", "<i8"), ("numel", "<i4"),
                          ("weight_decay", "<f4"), ("lr_scale", "<f4"), ("pad", "<i4")])


def tasks_to_device(tasks: list[tuple], device: torch.device) -> torch.Tensor:
    """``[(offset, numel, peer, flag)]`` or ``[(offset, numel, peer, flag, src_offset)]`` -> device byte tensor laid
    out as ``CopyTask[]`` (without a source offset the chunk sits at the same offset on both sides)."""
    arr = np.zeros(len(tasks), dtype=COPY_TASK_DTYPE)
    for i, t in enumerate(tasks):
        off, n, peer, flag = t[:4]
        arr[i] = (off, t[4] if len(t) > 4 else off, n, peer, 0, flag, 0)
    return torch.from_numpy(arr.view(np.uint8).copy()).to(device)


def segments_to_device(segs: list[tuple[int, int, int, int, float, float]], device: torch.device) -> torch.Tensor:
    """``[(grad_off, param_off, shard_off, numel, weight_decay, lr_scale)]`` -> device byte tensor of ``Segment[]``."""
    arr = np.zeros(len(segs), dtype=SEGMENT_DTYPE)
    for i, (go, po, so, n, wd, ls) in enumerate(segs):
        arr[i] = (go, po, so, n, wd, ls, 0)
    return torch.from_numpy(arr.view(np.uint8).copy()).to(device)
