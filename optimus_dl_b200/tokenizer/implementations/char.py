"""``char_tokenize``: UTF-8 bytes as tokens, BOS = 256, EOS = 257
(optimus_dl/modules/tokenizer/implementations/char.py)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .. import register_tokenizer
from ..base import BaseTokenizer
from ..config import BaseTokenizerConfig


@dataclass
class CharTokenizerConfig(BaseTokenizerConfig):
    pass


@register_tokenizer("char_tokenize", CharTokenizerConfig)
class CharTokenizer(BaseTokenizer):
    BOS, EOS = 256, 257

    def __init__(self, config, **kwargs: Any):
        super().__init__(config)

    def encode(self, text: str) -> list[int]:
        ids = list(text.encode("utf-8"))
        if self.config.add_bos:
            ids.insert(0, self.BOS)
        if self.config.add_eos:
            ids.append(self.EOS)
        return ids

    def decode(self, ids: list[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    @property
    def vocab_size(self) -> int:
        return 258

    @property
    def bos_token_id(self) -> int:
        return self.BOS

    @property
    def eos_token_id(self) -> int:
        return self.EOS
