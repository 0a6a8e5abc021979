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
    vocab_size: int = 256        # byte values; the two special ids follow
    bos_token_id: int = 256
    eos_token_id: int = 257


@register_tokenizer("char_tokenize", CharTokenizerConfig)
class CharTokenizer(BaseTokenizer):
    """UTF-8 bytes as tokens; the special ids and the reported vocabulary size come from the config
    (optimus_dl/modules/tokenizer/implementations/char.py)."""

    def __init__(self, config, **kwargs: Any):
        super().__init__(config)

    def encode(self, text: str) -> list[int]:
        ids = list(text.encode("utf-8"))
        if self.config.add_bos:
            if self.bos_token_id is None:
                raise ValueError("Tokenizer does not have a BOS token ID, but add_bos is True.")
            ids.insert(0, self.bos_token_id)
        if self.config.add_eos:
            if self.eos_token_id is None:
                raise ValueError("Tokenizer does not have an EOS token ID, but add_eos is True.")
            ids.append(self.eos_token_id)
        return ids

    def decode(self, ids: list[int]) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    @property
    def vocab_size(self) -> int:
        return max(int(self.config.vocab_size), int(self.config.eos_token_id or 0) + 1, int(self.config.bos_token_id or 0) + 1)

    @property
    def bos_token_id(self) -> int | None:
        return self.config.bos_token_id

    @property
    def eos_token_id(self) -> int | None:
        return self.config.eos_token_id
