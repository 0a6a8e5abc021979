"""Rank topology and collectives behind one small interface.

``Collective`` is the only thing the rest of the framework asks about ranks or uses to
communicate on the host-controlled path. ``FakeCollective`` serves single-process runs;
``MeshCollective`` wraps ``torch.distributed`` (NCCL for CUDA devices, Gloo otherwise) and lays
ranks out on two meshes exactly like the reference (optimus_dl/modules/distributed/mesh.py:86-163):

* parallel mesh ``(dp_replicate, dp_shard, tp)`` with ``tp`` innermost,
* physical mesh ``(nodes, local_ranks)``.

``sharding_world_size=None`` means "shard inside a node": ``local_world_size // tp_size``.
The in-kernel NVLink data plane (peer loads/stores on symmetric buffers) lives in
``parallel/symm.py`` and uses a Collective only to bootstrap.
"""

from __future__ import annotations

import datetime
import logging
import os
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, NamedTuple

import torch
import torch.distributed as dist

from ..core import env

logger = logging.getLogger(__name__)
ReduceOp = dist.ReduceOp


@dataclass
class DistributedConfig:
    """``tp_size`` = tensor-parallel degree; ``sharding_world_size`` = FSDP shard group size
    (``None``: ranks of one node divided by ``tp_size``)."""

    tp_size: int = 1
    sharding_world_size: int | None = 1


class Collective(ABC):
    """Topology properties plus the collectives the host-side code needs."""

    @property
    @abstractmethod
    def rank(self) -> int: ...

    @property
    @abstractmethod
    def world_size(self) -> int: ...

    @property
    @abstractmethod
    def local_rank(self) -> int: ...

    @property
    def is_master(self) -> bool:
        return self.rank == 0

    @property
    def is_local_master(self) -> bool:
        return self.local_rank == 0

    @property
    def tp_rank(self) -> int:
        return 0

    @property
    def tp_world_size(self) -> int:
        return 1

    @property
    def dp_rank(self) -> int:
        return self.rank // self.tp_world_size

    @property
    def dp_world_size(self) -> int:
        return self.world_size // self.tp_world_size

    @property
    @abstractmethod
    def default_device(self) -> torch.device: ...

    @property
    def process_group(self) -> Any:
        return None

    @property
    def local(self) -> "Collective":
        return self

    @property
    def tp_world(self) -> "Collective":
        return self

    @abstractmethod
    def barrier(self) -> None: ...

    @abstractmethod
    def all_reduce(self, tensor: torch.Tensor, op: Any = ReduceOp.SUM) -> None: ...

    @abstractmethod
    def all_gather(self, output: torch.Tensor, input: torch.Tensor) -> None: ...

    @abstractmethod
    def all_gather_to_list(self, input: torch.Tensor) -> list[torch.Tensor]: ...

    @abstractmethod
    def all_gather_objects(self, obj: Any) -> list[Any]: ...

    @abstractmethod
    def broadcast(self, tensor: torch.Tensor, src: int = 0) -> None: ...

    @abstractmethod
    def broadcast_objects(self, objects: list[Any], src: int = 0) -> None: ...

    def close(self) -> None:
        pass


def _best_single_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", 0)
    if getattr(torch.backends, "mps", None) is not None and torch.backends.mps.is_available():
        return torch.device("mps")
    return torch.device("cpu")


class FakeCollective(Collective):
    """World of one: every collective is the identity (optimus_dl/modules/distributed/fake.py:16-157)."""

    def __init__(self, rank: int = 0, world_size: int = 1, device: torch.device | None = None):
        assert world_size == 1, "FakeCollective only models a single process"
        self._rank = rank
        self._device = device

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def world_size(self) -> int:
        return 1

    @property
    def local_rank(self) -> int:
        return 0

    @property
    def default_device(self) -> torch.device:
        return self._device if self._device is not None else _best_single_device()

    def barrier(self) -> None:
        pass

    def all_reduce(self, tensor: torch.Tensor, op: Any = ReduceOp.SUM) -> None:
        pass

    def all_gather(self, output: torch.Tensor, input: torch.Tensor) -> None:
        output.view(-1)[: input.numel()].copy_(input.reshape(-1))

    def all_gather_to_list(self, input: torch.Tensor) -> list[torch.Tensor]:
        return [input.clone()]

    def all_gather_objects(self, obj: Any) -> list[Any]:
        return [obj]

    def broadcast(self, tensor: torch.Tensor, src: int = 0) -> None:
        pass

    def broadcast_objects(self, objects: list[Any], src: int = 0) -> None:
        pass


class Meshes(NamedTuple):
    """The two device meshes of a run (optimus_dl/modules/distributed/mesh.py:29-38): ``parallel_mesh`` with dimensions
    ``(dp_replicate, dp_shard, tp)`` and ``physical_mesh`` with ``(nodes, local_ranks)``."""

    parallel_mesh: Any
    physical_mesh: Any


class MeshCollective(Collective):
    """``torch.distributed`` backed collective with (dp_replicate, dp_shard, tp) topology."""

    def __init__(self, rank: int, world_size: int, local_world_size: int, local_rank: int,
                 device_type: str = "cuda", mesh: Any = None, process_group: Any = None, tp_size: int | None = None,
                 sharding_world_size: int | None = None, *, config: DistributedConfig | None = None,
                 timeout_s: float | None = None, _group: Any = None, _parent: "MeshCollective | None" = None):
        """Positional order and the ``tp_size`` / ``sharding_world_size`` / ``process_group`` keywords are those of
        optimus_dl/modules/distributed/mesh.py:66-77; ``config`` carries the same two sizes (explicit keywords win).
        A prebuilt ``mesh`` is not taken: the meshes are derived from the sizes."""
        if mesh is not None:
            raise NotImplementedError("MeshCollective builds its own device meshes; pass tp_size / sharding_world_size")
        if config is None:      # the keyword form: an absent sharding size means the node's ranks divided by tp_size
            cfg = DistributedConfig(tp_size=int(tp_size or 1), sharding_world_size=sharding_world_size) \
                if (tp_size is not None or sharding_world_size is not None) else DistributedConfig()
        else:
            cfg = config
            if tp_size is not None or sharding_world_size is not None:
                cfg = DistributedConfig(tp_size=int(tp_size if tp_size is not None else cfg.tp_size),
                                        sharding_world_size=sharding_world_size if sharding_world_size is not None
                                        else cfg.sharding_world_size)
        if process_group is not None and _group is None:
            _group = process_group
        self._rank, self._world, self._local_rank, self._local_world = rank, world_size, local_rank, local_world_size
        self._device_type = device_type
        self.config = cfg
        self._tp = max(1, int(cfg.tp_size))
        if world_size % self._tp != 0:
            raise ValueError(f"world size {world_size} is not divisible by tp_size {self._tp}")
        shard = cfg.sharding_world_size
        if shard is None:
            shard = max(1, local_world_size // self._tp)
        if (world_size // self._tp) % shard != 0:
            raise ValueError(f"dp world {world_size // self._tp} is not divisible by sharding_world_size {shard}")
        self._shard = shard
        self._replicate = world_size // (shard * self._tp)
        self._group = _group
        self._parent = _parent
        self._local_sub: MeshCollective | None = None
        self._tp_sub: MeshCollective | None = None
        self._parallel_mesh = self._physical_mesh = None
        if _parent is None:
            if not dist.is_initialized():
                backend = "nccl" if device_type == "cuda" else "gloo"
                kwargs: dict[str, Any] = {}
                if timeout_s is not None:
                    kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
                if device_type == "cuda":
                    torch.cuda.set_device(local_rank)
                    kwargs["device_id"] = torch.device("cuda", local_rank)
                dist.init_process_group(backend=backend, rank=rank, world_size=world_size, **kwargs)
            from torch.distributed.device_mesh import init_device_mesh

            self._parallel_mesh = init_device_mesh(device_type, (self._replicate, self._shard, self._tp),
                                                   mesh_dim_names=("dp_replicate", "dp_shard", "tp"))
            nodes = max(1, world_size // local_world_size)
            self._physical_mesh = init_device_mesh(device_type, (nodes, world_size // nodes),
                                                   mesh_dim_names=("nodes", "local_ranks"))
        else:
            self._parallel_mesh, self._physical_mesh = _parent._parallel_mesh, _parent._physical_mesh

    # topology ---------------------------------------------------------------
    @property
    def rank(self) -> int:
        return self._rank

    @property
    def world_size(self) -> int:
        return self._world

    @property
    def local_rank(self) -> int:
        return self._local_rank

    @property
    def tp_rank(self) -> int:
        root = self._parent or self
        return root._rank % root._tp

    @property
    def tp_world_size(self) -> int:
        return (self._parent or self)._tp

    @property
    def dp_rank(self) -> int:
        root = self._parent or self
        return root._rank // root._tp

    @property
    def dp_world_size(self) -> int:
        root = self._parent or self
        return root._world // root._tp

    @property
    def default_device(self) -> torch.device:
        if self._device_type == "cuda":
            return torch.device("cuda", self._local_rank)
        return torch.device(self._device_type)

    @property
    def process_group(self) -> Any:
        return self._group if self._group is not None else dist.group.WORLD

    @property
    def parallel_mesh(self):
        return self._parallel_mesh

    @property
    def meshes(self) -> "Meshes":
        return Meshes(self._parallel_mesh, self._physical_mesh)

    @property
    def physical_mesh(self):
        return self._physical_mesh

    @property
    def tp_mesh(self):
        return self._parallel_mesh["tp"]

    @property
    def dp_mesh(self):
        return self._parallel_mesh["dp_replicate", "dp_shard"]

    @property
    def dp_shard_mesh(self):
        return self._parallel_mesh["dp_shard"]

    @property
    def shard_world_size(self) -> int:
        return (self._parent or self)._shard

    @property
    def replicate_world_size(self) -> int:
        return (self._parent or self)._replicate

    @property
    def local(self) -> "MeshCollective":
        root = self._parent or self
        if root._local_sub is None:
            g = root._physical_mesh.get_group("local_ranks")
            root._local_sub = MeshCollective(dist.get_rank(g), dist.get_world_size(g), root._local_world,
                                             root._local_rank, root._device_type, config=root.config, _group=g,
                                             _parent=root)
        return root._local_sub

    @property
    def tp_world(self) -> "MeshCollective":
        root = self._parent or self
        if root._tp_sub is None:
            g = root._parallel_mesh.get_group("tp")
            root._tp_sub = MeshCollective(dist.get_rank(g), dist.get_world_size(g), root._local_world,
                                          root._local_rank, root._device_type, config=root.config, _group=g,
                                          _parent=root)
        return root._tp_sub

    # collectives --------------------------------------------------------------
    def barrier(self) -> None:
        if self._device_type == "cuda":
            dist.barrier(group=self.process_group, device_ids=[self._local_rank])
        else:
            dist.barrier(group=self.process_group)

    def all_reduce(self, tensor: torch.Tensor, op: Any = ReduceOp.SUM) -> None:
        dist.all_reduce(tensor, op=op, group=self.process_group)

    def all_gather(self, output: torch.Tensor, input: torch.Tensor) -> None:
        dist.all_gather_into_tensor(output, input.contiguous(), group=self.process_group)

    def all_gather_to_list(self, input: torch.Tensor) -> list[torch.Tensor]:
        out = [torch.empty_like(input) for _ in range(self.world_size)]
        dist.all_gather(out, input.contiguous(), group=self.process_group)
        return out

    def all_gather_objects(self, obj: Any) -> list[Any]:
        out: list[Any] = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.process_group)
        return out

    def broadcast(self, tensor: torch.Tensor, src: int = 0) -> None:
        dist.broadcast(tensor, src=dist.get_global_rank(self.process_group, src) if self._group is not None else src,
                       group=self.process_group)

    def broadcast_objects(self, objects: list[Any], src: int = 0) -> None:
        dist.broadcast_object_list(objects, src=dist.get_global_rank(self.process_group, src) if self._group is not None else src,
                                   group=self.process_group)

    def close(self) -> None:
        if self._parent is None and dist.is_initialized():
            try:
                self.barrier()
            finally:
                dist.destroy_process_group()


_collective: Collective | None = None


def reset_collective() -> None:
    """Forget the process-global collective (tests)."""
    global _collective
    _collective = None


def build_best_collective(config: DistributedConfig | Any = None, device: torch.device | None = None) -> Collective:
    """Process-global collective: Mesh when launched by torchrun with WORLD_SIZE > 1, else Fake
    (optimus_dl/modules/distributed/__init__.py:17-71)."""
    global _collective
    if _collective is not None:
        return _collective
    if config is not None and not isinstance(config, DistributedConfig):
        config = DistributedConfig(tp_size=int(config.get("tp_size", 1)),
                                   sharding_world_size=config.get("sharding_world_size", 1))
    needed = ("LOCAL_RANK", "LOCAL_WORLD_SIZE", "RANK", "WORLD_SIZE")
    if all(k in os.environ for k in needed) and env.get_world_size() > 1:
        dtype = (device.type if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        _collective = MeshCollective(env.get_rank(), env.get_world_size(), env.get_local_world_size(),
                                     env.get_local_rank(), dtype, config=config)
    else:
        _collective = FakeCollective(0, 1, device)
    return _collective
