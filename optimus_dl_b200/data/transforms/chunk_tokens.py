"""``chunk_tokens``: split long documents into pieces of at most ``max_seq_len`` (+1 for the label
shift) tokens (optimus_dl/modules/data/transforms/chunk_tokens.py:17-100)."""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from torchdata.nodes import BaseNode

from ...core.registry import RegistryConfigStrict
from . import register_transform
from .base import BaseTransform, adopt_saved_cfg


@dataclass
class ChunkTransformConfig(RegistryConfigStrict):
    max_seq_len: int = 1024
    add_one_for_shift: bool = True
    max_chunks: int | None = None
    field: str = "input_ids"


class ChunkTokensNode(BaseNode):
    """State under the reference's keys: ``buffer`` holds what is left of the current document, ``cfg`` the
    configuration, ``source_state`` the upstream state (``rest``, the document's other fields, is this package's
    addition: the reference drops them)."""

    def __init__(self, node: BaseNode, cfg: Any):
        super().__init__()
        self.node, self.cfg = node, cfg
        self.buffer: Any = []
        self.rest: dict[str, Any] = {}

    def reset(self, initial_state: dict | None = None):
        super().reset(initial_state)
        self.buffer, self.rest = [], {}
        if initial_state:
            self.buffer = copy.deepcopy(initial_state.get("buffer", []))
            self.rest = copy.deepcopy(initial_state.get("rest", {}))
            self.cfg = adopt_saved_cfg(self.cfg, initial_state.get("cfg"))
            self.node.reset(initial_state["source_state"])
        else:
            self.node.reset()

    def get_state(self) -> dict[str, Any]:
        return copy.deepcopy({"buffer": self.buffer, "cfg": self.cfg, "source_state": self.node.state_dict(),
                              "rest": self.rest})

    def next(self) -> dict[str, Any]:
        size = int(self.cfg.max_seq_len) + (1 if self.cfg.add_one_for_shift else 0)
        while len(self.buffer) == 0:                       # empty documents give no chunk
            item = next(self.node)
            self.buffer = item[self.cfg.field]
            if self.cfg.max_chunks is not None:
                self.buffer = self.buffer[: int(self.cfg.max_chunks) * size]
            self.rest = {k: v for k, v in item.items() if k != self.cfg.field}
        chunk, self.buffer = self.buffer[:size], self.buffer[size:]
        return {**self.rest, self.cfg.field: chunk}


@register_transform("chunk_tokens", ChunkTransformConfig)
class ChunkTransform(BaseTransform):
    def build(self, source: BaseNode) -> BaseNode:
        return ChunkTokensNode(source, self.cfg)


ChunkTransformNode = ChunkTokensNode   # the reference's name
