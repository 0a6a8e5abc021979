"""``to_device``: numpy -> tensors, pin, asynchronous host-to-device copy, small prefetch so the copy
of batch i+1 overlaps the compute of batch i (optimus_dl/modules/data/transforms/to_device.py:21-119)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import numpy as np
import torch
from torchdata.nodes import BaseNode, Mapper, PinMemory, Prefetcher

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform


@dataclass
class ToDeviceTransformConfig(RegistryConfigStrict):
    device: str | None = None
    pin_memory: bool = True
    prefetch_factor: int = 2
    non_blocking: bool = True
    # the reference's fields (optimus_dl/modules/data/transforms/to_device.py:22-33)
    properties: list[str] | None = None        # keys to convert and move; None = every value
    pin_prefetch_factor: int | None = None     # same role as prefetch_factor; wins when set
    pin_snapshot_frequency: int = 128


def _to_tensor(batch: Any) -> Any:
    if isinstance(batch, dict):
        return {k: _to_tensor(v) for k, v in batch.items()}
    if isinstance(batch, np.ndarray):
        if batch.dtype in (np.uint16, np.uint32, np.uint64):
            # token files are stored unsigned; index-taking ops (embedding, gather) want signed 64-bit
            batch = batch.astype(np.int64)
        return torch.from_numpy(np.ascontiguousarray(batch))
    return batch


class _StatelessMap(BaseNode):
    """``fn`` applied to every item; the state IS the source's state (no ``source`` level of its own)."""

    def __init__(self, source: BaseNode, fn: Any):
        super().__init__()
        self.source, self.fn = source, fn

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self.source.reset(initial_state)

    def get_state(self) -> dict[str, Any]:
        return self.source.state_dict()

    def next(self) -> Any:
        return self.fn(next(self.source))


class _Mover:
    def __init__(self, device: torch.device, non_blocking: bool):
        self.device, self.non_blocking = device, non_blocking

    def __call__(self, batch: Any) -> Any:
        if isinstance(batch, dict):
            return {k: self(v) for k, v in batch.items()}
        if isinstance(batch, torch.Tensor):
            return batch.to(self.device, non_blocking=self.non_blocking)
        return batch


@register_transform("to_device", ToDeviceTransformConfig)
class ToDeviceTransform(BaseTransform):
    def __init__(self, cfg, device: Any = None, **kwargs: Any):
        super().__init__(cfg)
        dev = cfg.device if cfg.device is not None else device
        self.device = torch.device(dev) if dev is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.properties = list(cfg.properties) if cfg.properties is not None else None

    def _map(self, sample: Any) -> Any:
        """Convert and move one sample in the calling thread. With ``properties`` set, only those keys are touched
        (lists among them become tensors); without, every array / tensor value moves."""
        if isinstance(sample, dict) and self.properties is not None:
            out = dict(sample)
            for k in self.properties:
                if k in out:
                    v = _to_tensor(out[k])
                    if not isinstance(v, (torch.Tensor, dict)):
                        v = torch.as_tensor(v)
                    out[k] = _Mover(self.device, bool(self.cfg.non_blocking))(v)
            return out
        return _Mover(self.device, bool(self.cfg.non_blocking))(_to_tensor(sample))

    def build(self, source: BaseNode) -> BaseNode:
        """CPU: one ``Mapper``. CUDA: ``PinMemory`` -> ``Mapper`` (asynchronous copy) -> ``Prefetcher``, the chain of
        optimus_dl/modules/data/transforms/to_device.py:92-119; the conversion of numpy arrays to tensors that has to
        precede pinning (``PinMemory`` leaves arrays as they are) is a node that adds no level to the checkpointed
        state, so states nest alike in both code bases."""
        props = list(self.properties) if self.properties is not None else None
        if props is None:
            convert = _to_tensor
        else:
            convert = lambda b, _p=frozenset(props): ({k: (_to_tensor(v) if k in _p else v) for k, v in b.items()}  # noqa: E731
                                                      if isinstance(b, dict) else _to_tensor(b))
        depth = self.cfg.pin_prefetch_factor if self.cfg.pin_prefetch_factor is not None else self.cfg.prefetch_factor
        if self.device.type == "cpu":
            node: BaseNode = Mapper(source, convert)
        elif self.device.type != "cuda":
            mover = _Mover(self.device, False)
            node = Mapper(source, lambda b: mover(convert(b)))
        else:
            node = _StatelessMap(source, convert)
            if self.cfg.pin_memory:
                node = PinMemory(node, pin_memory_device="cuda", snapshot_frequency=int(self.cfg.pin_snapshot_frequency))
            node = Mapper(node, _Mover(self.device, bool(self.cfg.non_blocking)))
            if depth and depth > 0:
                node = Prefetcher(node, prefetch_factor=int(depth), snapshot_frequency=int(self.cfg.pin_snapshot_frequency))
        return node
