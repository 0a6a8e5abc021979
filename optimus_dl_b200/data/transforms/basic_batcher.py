"""``basic_batcher``: group whole documents, pad to the longest (or flatten)
(optimus_dl/modules/data/transforms/basic_batcher.py:18-268).

A batch closes at ``batch_size`` items or when the next item would exceed ``max_tokens`` (that item
is kept for the next batch; a single over-long item still forms a batch of its own). Padded
output: the token field ``(B, max_len)``, ``seq_lens``, ``position_ids`` (0 on padding), ``document_ids``
(row index, or ``None`` when ``add_document_ids`` is off). Flattened output additionally carries
shifted ``labels``, ``cu_seqlens`` and ``max_seqlen``. Works on lists, numpy arrays and tensors.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

import numpy as np
import torch
from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform


@dataclass
class BasicBatcherConfig(RegistryConfigStrict):
    batch_size: int | None = None
    max_tokens: int | None = None
    pad_token_id: int = "???"  # type: ignore[assignment]
    field: str = "input_ids"
    flatten: bool = False
    add_document_ids: bool = True


class BasicBatcherNode(BaseNode):
    def __init__(self, node: BaseNode, cfg: Any):
        super().__init__()
        if cfg.batch_size is None and cfg.max_tokens is None:
            raise ValueError("Either batch_size or max_tokens must be specified in BasicBatcherConfig.")
        self.node, self.cfg = node, cfg
        self._peeked: Any = None

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self._peeked = None
        if initial_state:
            self._peeked = copy.deepcopy(initial_state.get("_peeked_item"))
            self.node.reset(initial_state["source_state"])
        else:
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        return {"cfg": copy.deepcopy(self.cfg), "source_state": self.node.state_dict(), "_peeked_item": copy.deepcopy(self._peeked)}

    def _collect(self) -> list[dict]:
        items: list[dict] = []
        tokens = 0
        while self.cfg.batch_size is None or len(items) < self.cfg.batch_size:
            try:
                if self._peeked is not None:
                    item, self._peeked = self._peeked, None
                else:
                    item = next(self.node)
            except StopIteration:
                if not items:
                    raise
                break
            n = len(item[self.cfg.field])
            if self.cfg.max_tokens is not None and tokens + n > self.cfg.max_tokens and items:
                self._peeked = item
                break
            items.append(item)
            tokens += n
        return items

    def next(self) -> dict[str, Any]:
        items = self._collect()
        f = self.cfg.field
        seqs = [it[f] for it in items]
        as_torch = isinstance(seqs[0], torch.Tensor)
        if not as_torch:
            seqs = [np.asarray(s) for s in seqs]
        lens = [len(s) for s in seqs]
        B = len(seqs)
        docs_on = bool(self.cfg.add_document_ids)
        if self.cfg.flatten:
            sl = [n - 1 for n in lens]
            if as_torch:
                dev = seqs[0].device
                ids = torch.cat([s[:-1] for s in seqs])
                return {f: ids[None], "labels": torch.cat([s[1:] for s in seqs])[None],
                        "position_ids": torch.cat([torch.arange(n, device=dev) for n in sl])[None],
                        "document_ids": torch.cat([torch.full((n,), i, device=dev, dtype=torch.long)
                                                   for i, n in enumerate(sl)])[None] if docs_on else None,
                        "seq_lens": torch.tensor([len(ids)], device=dev),
                        "cu_seqlens": torch.cumsum(torch.tensor([0] + sl, device=dev), 0).to(torch.int32),
                        "max_seqlen": int(max(sl))}
            ids = np.concatenate([s[:-1] for s in seqs]).astype(np.int64)
            return {f: ids[None], "labels": np.concatenate([s[1:] for s in seqs]).astype(np.int64)[None],
                    "position_ids": np.concatenate([np.arange(n) for n in sl]).astype(np.int64)[None],
                    "document_ids": np.concatenate([np.full(n, i) for i, n in enumerate(sl)]).astype(np.int64)[None]
                    if docs_on else None,
                    "seq_lens": np.array([len(ids)], dtype=np.int64),
                    "cu_seqlens": np.cumsum([0] + sl).astype(np.int32), "max_seqlen": int(max(sl))}
        L = max(lens)
        if as_torch:
            dev = seqs[0].device
            out = torch.full((B, L), self.cfg.pad_token_id, device=dev, dtype=seqs[0].dtype)
            for i, s in enumerate(seqs):
                out[i, : lens[i]] = s
            blens = torch.tensor(lens, dtype=torch.long, device=dev)
            pos = torch.arange(L, device=dev).unsqueeze(0).expand(B, -1).clone()
            pos[pos >= blens.unsqueeze(1)] = 0
            docs = torch.arange(B, device=dev).unsqueeze(1).expand(-1, L) if docs_on else None
        else:
            out = np.full((B, L), self.cfg.pad_token_id, dtype=np.int64)
            for i, s in enumerate(seqs):
                out[i, : lens[i]] = s
            blens = np.array(lens, dtype=np.int64)
            pos = np.tile(np.arange(L), (B, 1))
            pos[np.arange(L)[None, :] >= blens[:, None]] = 0
            docs = (np.arange(B)[:, None] * np.ones((1, L), dtype=np.int64)) if docs_on else None
        return {f: out, "seq_lens": blens, "position_ids": pos, "document_ids": docs}


@register_transform("basic_batcher", BasicBatcherConfig)
class BasicBatcher(BaseTransform):
    def build(self, source: BaseNode) -> BaseNode:
        return BasicBatcherNode(source, self.cfg)
