"""``tokenize``: text -> token ids with a registry tokenizer through a parallel mapper
(optimus_dl/modules/data/transforms/tokenize.py:27-103)."""

from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any

from torchdata.nodes import BaseNode, ParallelMapper

from ...core.registry import RegistryConfig
from ...tokenizer import build_tokenizer       # module-level so that callers can substitute the factory
from . import register_transform
from .base import BaseTransform, MapperConfig

logger = logging.getLogger(__name__)


@dataclass
class TokenizeTransformConfig(RegistryConfig):
    tokenizer_config: Any = None
    worker_cfg: MapperConfig = field(default_factory=MapperConfig)
    input_field: str = "text"
    output_field: str = "input_ids"
    keep_text: bool = False
    debug_samples: int = 0          # log this many tokenised samples (text and ids) for inspection


class _Tokenize:
    """Picklable callable; the tokenizer is built lazily inside each worker."""

    def __init__(self, tok_cfg: Any, in_f: str, out_f: str, keep: bool, debug_samples: int = 0):
        self.tok_cfg, self.in_f, self.out_f, self.keep = tok_cfg, in_f, out_f, keep
        self.debug_samples, self._shown = int(debug_samples), 0
        self._tok = None

    def __call__(self, item: dict) -> dict:
        if self._tok is None:
            self._tok = build_tokenizer(self.tok_cfg)
        out = dict(item) if self.keep else {k: v for k, v in item.items() if k != self.in_f}
        out[self.out_f] = self._tok.encode(item[self.in_f])
        if self._shown < self.debug_samples:
            self._shown += 1
            logger.info("tokenize sample %d: %r -> %s", self._shown, str(item[self.in_f])[:200], list(out[self.out_f])[:64])
        return out

    def __getstate__(self):
        return {"tok_cfg": self.tok_cfg, "in_f": self.in_f, "out_f": self.out_f, "keep": self.keep, "_tok": None,
                "debug_samples": self.debug_samples, "_shown": self._shown}


@register_transform("tokenize", TokenizeTransformConfig)
class TokenizeTransform(BaseTransform):
    def __init__(self, cfg, **kwargs: Any):
        super().__init__(cfg)

    def _callable(self) -> _Tokenize:
        from ...core import conf

        tok_cfg = conf.to_container(self.cfg.tokenizer_config, resolve=True) if conf.is_config(self.cfg.tokenizer_config) \
            else self.cfg.tokenizer_config
        return _Tokenize(tok_cfg, self.cfg.input_field, self.cfg.output_field, bool(self.cfg.keep_text),
                         int(self.cfg.get("debug_samples", 0) or 0))

    def _map(self, item: dict) -> dict:
        """Tokenise one sample in this process (what the mapper node calls per item)."""
        if getattr(self, "_fn", None) is None:
            self._fn = self._callable()
        return self._fn(item)

    def build(self, source: BaseNode) -> BaseNode:
        """Always a ``ParallelMapper`` with the configured worker settings (it maps inline when ``num_workers`` is 0), as
        optimus_dl/modules/data/transforms/tokenize.py:97-103 builds it: the node's checkpointed state then nests
        the same way in both code bases."""
        w = self.cfg.worker_cfg
        return ParallelMapper(source=source, map_fn=self._callable(), num_workers=int(w.num_workers),
                              in_order=bool(w.in_order), method=w.method, snapshot_frequency=int(w.snapshot_frequency),
                              prebatch=w.prebatch)
