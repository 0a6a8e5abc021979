"""``tokenized_flat``: memory-maps raw token files as one stream, gives every rank an equal token
span and yields ready ``(batch_size, seq_len)`` blocks in the files' dtype
(optimus_dl/modules/data/datasets/tokenized_flat_dataset.py:17-173: same shapes, same stop rule -- a block that ends
past the rank's span is dropped -- and the same state keys). ``add_one_for_shift: true`` is an addition: rows of
``seq_len + 1`` tokens that overlap by one, so that shifting inputs against targets loses no token."""

from __future__ import annotations

import glob
import os
from dataclasses import dataclass
from typing import Any

import numpy as np

from ...core.registry import RegistryConfigStrict
from . import register_dataset
from .base import BaseDataset


@dataclass
class TokenizedFlatDatasetConfig(RegistryConfigStrict):
    files: Any = "???"              # path, glob or list of paths
    dtype: str = "uint16"
    batch_size: int = 1
    seq_len: int = 1024
    header_bytes: int = 0
    offset: int | None = None       # the reference's name for header_bytes (bytes skipped at the start of raw files)
    add_one_for_shift: bool = False


@register_dataset("tokenized_flat", TokenizedFlatDatasetConfig)
class TokenizedFlatDataset(BaseDataset):
    def __init__(self, cfg, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        super().__init__(cfg, rank, world_size, seed)
        files = cfg.files
        if isinstance(files, str):
            files = sorted(glob.glob(os.path.expanduser(files))) or [os.path.expanduser(files)]
        self.files = list(files)
        self.maps = []
        for f in self.files:
            if f.endswith(".npy"):
                self.maps.append(np.load(f, mmap_mode="r"))
            else:
                skip = cfg.offset if cfg.offset is not None else cfg.header_bytes
                name = str(cfg.dtype)
                name = name[3:] if name.startswith("np.") else name        # "np.uint16" and "uint16" both name the type
                self.maps.append(np.memmap(f, dtype=np.dtype(name), mode="r", offset=int(skip)))
        self.cum = np.concatenate([[0], np.cumsum([len(m) for m in self.maps])]).astype(np.int64)
        total = int(self.cum[-1])
        per = total // world_size
        self.start, self.end = rank * per, (rank + 1) * per
        self.block = int(cfg.batch_size) * int(cfg.seq_len)
        self.pos = self.start

    def _read(self, a: int, b: int) -> np.ndarray:
        out = np.empty(b - a, dtype=self.maps[0].dtype)
        o = 0
        f = int(np.searchsorted(self.cum, a, side="right") - 1)
        while a < b:
            fe = int(self.cum[f + 1])
            take = min(b, fe)
            out[o:o + take - a] = self.maps[f][a - int(self.cum[f]): take - int(self.cum[f])]
            o += take - a
            a = take
            f += 1
        return out

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        st = initial_state or {}
        assert st.get("world_size", self.world_size) == self.world_size and st.get("rank", self.rank) == self.rank
        self.pos = int(st.get("index", st.get("pos", self.start)))
        self.end = int(st.get("limit", self.end))

    def get_state(self) -> dict[str, Any]:
        return {"files": list(self.files), "index": self.pos, "limit": self.end, "seq_len": int(self.cfg.seq_len),
                "batch_size": int(self.cfg.batch_size), "rank": self.rank, "world_size": self.world_size}

    def next(self) -> dict[str, Any]:
        B, T = int(self.cfg.batch_size), int(self.cfg.seq_len)
        total = int(self.cum[-1])
        if self.cfg.add_one_for_shift:
            if self.pos + self.block + 1 > self.end:
                raise StopIteration
            rows = [self._read(self.pos + i * T, self.pos + (i + 1) * T + 1) for i in range(B)]
            self.pos += self.block
            return {"input_ids": np.stack(rows)}
        if self.pos + self.block > total:
            raise StopIteration
        data = self._read(self.pos, self.pos + self.block)
        self.pos += self.block
        if self.pos > self.end:              # the block reached past this rank's span: dropped, the rank is done
            raise StopIteration
        return {"input_ids": data.reshape(B, T)}
