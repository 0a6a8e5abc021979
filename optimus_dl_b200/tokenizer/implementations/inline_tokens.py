"""``inline_tokens_tokenizer``: an explicit vocabulary matched greedily, longest token first, with a
policy for text no token covers (optimus_dl/modules/tokenizer/implementations/inline_tokens.py).
Ids: the listed tokens in order, then BOS, EOS and (with the ``unk`` policy) UNK."""

from __future__ import annotations

import enum
import re
from dataclasses import dataclass
from typing import Any

from .. import register_tokenizer
from ..base import BaseTokenizer
from ..config import BaseTokenizerConfig


class UnkStrategy(str, enum.Enum):
    IGNORE = "ignore"
    RAISE = "raise"
    UNK = "unk"


@dataclass
class InlineTokensTokenizerConfig(BaseTokenizerConfig):
    tokens: list[str] = "???"  # type: ignore[assignment]
    unk_strategy: UnkStrategy = UnkStrategy.RAISE


@register_tokenizer("inline_tokens_tokenizer", InlineTokensTokenizerConfig)
class InlineTokensTokenizer(BaseTokenizer):
    def __init__(self, config, **kwargs: Any):
        super().__init__(config)
        self.tokens = list(config.tokens)
        self._ids = {t: i for i, t in enumerate(self.tokens)}
        by_len = sorted(self.tokens, key=len, reverse=True)
        self._pattern = re.compile("(" + "|".join(re.escape(t) for t in by_len) + ")")
        n = len(self.tokens)
        self._bos, self._eos = n, n + 1
        strat = config.unk_strategy
        self.unk_strategy = strat if isinstance(strat, UnkStrategy) else UnkStrategy(str(strat).split(".")[-1].lower())
        self._unk = n + 2 if self.unk_strategy == UnkStrategy.UNK else None
        self._unk_token_id = self._unk
        self._vocab = n + 2 + (1 if self._unk is not None else 0)

    def encode(self, text: str) -> list[int]:
        ids = [self._bos] if self.config.add_bos else []
        for piece in self._pattern.split(text):
            if piece == "":
                continue
            if piece in self._ids:
                ids.append(self._ids[piece])
            elif self.unk_strategy == UnkStrategy.RAISE:
                raise ValueError(f"Unknown token/characters encountered: {piece!r} is not covered by the vocabulary")
            elif self.unk_strategy == UnkStrategy.UNK:
                ids.append(self._unk)
        if self.config.add_eos:
            ids.append(self._eos)
        return ids

    def decode(self, ids: list[int]) -> str:
        out = []
        for i in ids:
            if 0 <= i < len(self.tokens):
                out.append(self.tokens[i])
            elif self._unk is not None and i == self._unk:
                out.append("<UNK>")
            elif i not in (self._bos, self._eos):
                raise ValueError(f"Invalid token ID: {i}")
        return "".join(out)

    @property
    def vocab_size(self) -> int:
        return self._vocab

    @property
    def bos_token_id(self) -> int:
        return self._bos

    @property
    def eos_token_id(self) -> int:
        return self._eos
