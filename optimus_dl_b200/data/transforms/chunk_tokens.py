"""``chunk_tokens``: split long documents into pieces of at most ``max_seq_len`` (+1 for the label
shift) tokens (optimus_dl/modules/data/transforms/chunk_tokens.py:17-100)."""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform


@dataclass
class ChunkTransformConfig(RegistryConfigStrict):
    max_seq_len: int = 1024
    add_one_for_shift: bool = True
    max_chunks: int | None = None
    field: str = "input_ids"


class ChunkTokensNode(BaseNode):
    def __init__(self, node: BaseNode, cfg: Any):
        super().__init__()
        self.node, self.cfg = node, cfg
        self.pending: list = []

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        if initial_state:
            self.pending = copy.deepcopy(initial_state.get("pending", []))
            self.node.reset(initial_state["source_state"])
        else:
            self.pending = []
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        return {"pending": copy.deepcopy(self.pending), "source_state": self.node.state_dict()}

    def next(self) -> dict[str, Any]:
        while not self.pending:
            item = next(self.node)
            toks = item[self.cfg.field]
            size = int(self.cfg.max_seq_len) + (1 if self.cfg.add_one_for_shift else 0)
            chunks = [toks[i:i + size] for i in range(0, len(toks), size)]
            if self.cfg.max_chunks is not None:
                chunks = chunks[: int(self.cfg.max_chunks)]
            rest = {k: v for k, v in item.items() if k != self.cfg.field}
            self.pending = [{**rest, self.cfg.field: c} for c in chunks if len(c) > 0]
        return self.pending.pop(0)


@register_transform("chunk_tokens", ChunkTransformConfig)
class ChunkTransform(BaseTransform):
    def build(self, source: BaseNode) -> BaseNode:
        return ChunkTokensNode(source, self.cfg)


ChunkTransformNode = ChunkTokensNode   # the reference's name
