"""``tokenized_dataset``: reads shards written by the pretokenize recipe
(optimus_dl/modules/data/datasets/tokenized_dataset.py:27-311).

Layout: ``index.json`` lists shards; each shard is ``<name>_NNNNNNNNNN.npy`` (all tokens, one flat
array) plus ``<name>_NNNNNNNNNN_lens.npy`` (document lengths). Files are opened with
``np.load(mmap_mode="r")``. A pluggable sampling strategy decides which token ranges form an item.
Yields ``{"input_ids", "document_id", "seq_lens"}``. Resume requires the same rank / world size.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from ...core.registry import RegistryConfig
from . import register_dataset
from .base import BaseDataset
from .strategies import build_strategy


@dataclass
class TokenizedDatasetConfig(RegistryConfig):
    data_dir: str = "???"
    index_file: str = "index.json"
    strategy: Any = field(default_factory=lambda: {"_name": "document"})
    limit_documents: int | None = None
    limit: int | None = None        # the reference's name for limit_documents


@register_dataset("tokenized_dataset", TokenizedDatasetConfig)
class TokenizedDataset(BaseDataset):
    def __init__(self, cfg, rank: int = 0, world_size: int = 1, seed: int = 0, **kwargs: Any):
        super().__init__(cfg, rank, world_size, seed)
        with open(os.path.join(cfg.data_dir, cfg.index_file)) as f:
            self.index = json.load(f)
        self.shards = self.index["files"] if "files" in self.index else self.index["shards"]
        self._tokens: list[np.ndarray | None] = [None] * len(self.shards)
        lens = []
        self.shard_doc_start = [0]
        for sh in self.shards:
            l = np.load(os.path.join(cfg.data_dir, sh["lens_file"] if "lens_file" in sh else sh["lens"]), mmap_mode="r")
            lens.append(np.asarray(l, dtype=np.int64))
            self.shard_doc_start.append(self.shard_doc_start[-1] + len(l))
        self.doc_lens = np.concatenate(lens) if lens else np.zeros(0, dtype=np.int64)
        self.shard_num_docs = [len(l) for l in lens]
        limit = cfg.get("limit") if cfg.get("limit") is not None else cfg.get("limit_documents")
        if limit is not None:
            self.doc_lens = self.doc_lens[: int(limit)]
        self.total_docs = len(self.doc_lens)
        # tokens come back in the dtype the shards were written with (index.json: config.dtype; "np.uint16" and
        # "uint16" both name the type), batchers widen to int64
        name = str((self.index.get("config") or {}).get("dtype", "")) if isinstance(self.index, dict) else ""
        name = name[3:] if name.startswith("np.") else name
        self.dtype = np.dtype(name) if name else None
        self.shard_tok_start = [np.concatenate([[0], np.cumsum(l)]) for l in lens]
        self.strategy = build_strategy(cfg.strategy, rank=rank, world_size=world_size, seed=seed)
        # what all ranks must draw alike (shuffles, offsets) comes from the corpus-wide seed when the builder passes
        # one; ``seed`` itself may differ per rank
        self.strategy.global_seed = kwargs.get("global_seed")
        self.strategy.initialize(self.doc_lens)

    def _shard_tokens(self, s: int) -> np.ndarray:
        if self._tokens[s] is None:
            sh = self.shards[s]
            self._tokens[s] = np.load(os.path.join(self.cfg.data_dir, sh["file"] if "file" in sh else sh["tokens"]),
                                      mmap_mode="r")
        return self._tokens[s]

    def _read(self, doc: int, start: int, end: int) -> np.ndarray:
        s = int(np.searchsorted(self.shard_doc_start, doc, side="right") - 1)
        local = doc - self.shard_doc_start[s]
        base = int(self.shard_tok_start[s][local])
        toks = self._shard_tokens(s)
        if base + end > len(toks):
            raise RuntimeError(f"Data corruption: lens file does not match token file (shard {s}: document {local} ends "
                               f"at token {base + end}, the shard has {len(toks)}).")
        out = np.asarray(toks[base + start: base + end])
        if self.dtype is None:
            self.dtype = out.dtype
        return out if out.dtype == self.dtype else out.astype(self.dtype)

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        if initial_state:
            assert initial_state.get("rank", self.rank) == self.rank and \
                initial_state.get("world_size", self.world_size) == self.world_size, \
                "tokenized_dataset must be resumed with the same rank and world size"
            self.strategy.reset(initial_state["strategy_state"] if "strategy_state" in initial_state
                                else initial_state.get("strategy"))          # "strategy": this package's earlier key
        else:
            self.strategy.reset(None)

    def get_state(self) -> dict[str, Any]:
        """Keys of optimus_dl/modules/data/datasets/tokenized_dataset.py:299-311."""
        limit = self.cfg.get("limit") if self.cfg.get("limit") is not None else self.cfg.get("limit_documents")
        return {"rank": self.rank, "world_size": self.world_size, "strategy_state": self.strategy.get_state(),
                "data_dir": str(self.cfg.data_dir), "index_file": self.cfg.index_file, "limit": limit, "seed": self.seed}

    def next(self) -> dict[str, Any]:
        segs = self.strategy.next_segments()
        parts = [self._read(d, a, b) for d, a, b in segs]
        toks = np.concatenate(parts) if len(parts) > 1 else parts[0]
        doc_ids = np.concatenate([np.full(b - a, d, dtype=np.int64) for d, a, b in segs])
        return {"input_ids": toks, "document_id": doc_ids if len(segs) > 1 else int(segs[0][0]),
                "seq_lens": np.array([b - a for _, a, b in segs], dtype=np.int64)}
