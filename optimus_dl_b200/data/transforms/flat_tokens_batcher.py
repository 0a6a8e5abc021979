"""``flat_batcher``: pool the tokens of incoming documents and emit packed batches with labels
already shifted (optimus_dl/modules/data/transforms/flat_tokens_batcher.py:20-224).

Output: ``input_ids`` and ``labels`` of shape ``(B, T)`` — or ``(1, total)`` with ``flatten`` — and, with
``mask_documents``, ``position_ids`` (restarting per document), ``document_ids`` (renumbered from 0 inside
the batch) and for flat batches ``cu_seqlens`` (int32) and ``max_seqlen``. The label of the last
token of a document is never the first token of the next one: each document contributes
``tokens[:-1]`` as inputs and ``tokens[1:]`` as labels.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

import numpy as np
from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform, adopt_saved_cfg, MapperConfig, ProcessMapperConfig


@dataclass
class FlatTokensBatcherConfig(RegistryConfigStrict):
    batch_size: int | None = None
    seq_len: int | None = None
    max_tokens: int | None = None
    worker_cfg: MapperConfig = field(default_factory=ProcessMapperConfig)
    field: str = "input_ids"
    mask_documents: bool = False
    flatten: bool = False


class FlatTokensBatcherNode(BaseNode):
    # attribute -> key in the checkpointed state (the keys of
    # optimus_dl/modules/data/transforms/flat_tokens_batcher.py:109-121, so states are interchangeable)
    _BUFS = {"inputs": "input_buffer", "labels": "label_buffer", "positions": "position_ids_buffer",
             "docs": "document_ids_buffer"}

    def __init__(self, node: BaseNode, cfg: Any):
        super().__init__()
        self.node, self.cfg = node, cfg
        if cfg.flatten:
            if not cfg.mask_documents:
                raise ValueError("FlatTokensBatcher: 'mask_documents' must be True when 'flatten' is True. Flat "
                                 "batches need document tracking to produce 'cu_seqlens' and 'position_ids'.")
            if cfg.max_tokens is None and (cfg.batch_size is None or cfg.seq_len is None):
                raise ValueError("FlatTokensBatcher (flatten=True) requires either 'max_tokens' or both 'batch_size' "
                                 "and 'seq_len'.")
        elif cfg.batch_size is None or cfg.seq_len is None:
            raise ValueError("FlatTokensBatcher (flatten=False) requires 'batch_size' and 'seq_len'.")
        self._clear()

    def _clear(self) -> None:
        self.inputs: list[int] = []
        self.labels: list[int] = []
        self.positions: list[int] = []
        self.docs: list[int] = []
        self.next_doc = 0

    @property
    def target_size(self) -> int:
        if self.cfg.max_tokens is not None:
            return int(self.cfg.max_tokens)
        return int(self.cfg.batch_size) * int(self.cfg.seq_len)

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self._clear()
        if initial_state:
            for attr, key in self._BUFS.items():
                setattr(self, attr, list(initial_state.get(key, initial_state.get(attr, []))))
            self.next_doc = initial_state.get("_current_doc_id", initial_state.get("next_doc", 0))
            self.cfg = adopt_saved_cfg(self.cfg, initial_state.get("cfg"))
            self.node.reset(initial_state["source_state"])
        else:
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        st = {key: list(getattr(self, attr)) for attr, key in self._BUFS.items()}
        st.update(_current_doc_id=self.next_doc, cfg=self.cfg, source_state=self.node.state_dict())
        return copy.deepcopy(st)

    def next(self) -> dict[str, Any]:
        n = self.target_size
        track = bool(self.cfg.mask_documents)
        while len(self.inputs) < n:
            toks = next(self.node)[self.cfg.field]
            m = len(toks)
            if m <= 1:
                continue
            toks = toks.tolist() if hasattr(toks, "tolist") else list(toks)
            self.inputs.extend(toks[:-1])
            self.labels.extend(toks[1:])
            if track:
                self.positions.extend(range(m - 1))
                self.docs.extend([self.next_doc] * (m - 1))
                self.next_doc += 1
        shape = (1, -1) if self.cfg.flatten else (int(self.cfg.batch_size), -1)
        out = {"input_ids": np.asarray(self.inputs[:n], dtype=np.int64).reshape(shape),
               "labels": np.asarray(self.labels[:n], dtype=np.int64).reshape(shape)}
        del self.inputs[:n], self.labels[:n]
        if track:
            pos = np.asarray(self.positions[:n], dtype=np.int64)
            doc = np.asarray(self.docs[:n], dtype=np.int64)
            del self.positions[:n], self.docs[:n]
            _, doc = np.unique(doc, return_inverse=True)
            out["position_ids"] = pos.reshape(shape)
            out["document_ids"] = doc.reshape(shape).astype(np.int64)
            if self.cfg.flatten:
                starts = np.flatnonzero(np.diff(doc, prepend=-1) != 0)
                cu = np.append(starts, len(doc)).astype(np.int32)
                out["cu_seqlens"] = cu
                out["max_seqlen"] = int(np.diff(cu).max())
        return out


@register_transform("flat_batcher", FlatTokensBatcherConfig)
class FlatTokensBatcher(BaseTransform):
    def build(self, source: BaseNode) -> BaseNode:
        return FlatTokensBatcherNode(source, self.cfg)
