"""``tiktoken``: OpenAI BPE encodings; the end-of-text token serves as both BOS and EOS
(optimus_dl/modules/tokenizer/implementations/tiktoken.py)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .. import register_tokenizer
from ..base import BaseTokenizer
from ..config import BaseTokenizerConfig


@dataclass
class TiktokenConfig(BaseTokenizerConfig):
    name: str = "gpt2"


@register_tokenizer("tiktoken", TiktokenConfig)
class TiktokenTokenizer(BaseTokenizer):
    def __init__(self, config, **kwargs: Any):
        super().__init__(config)
        import tiktoken

        try:
            self.enc = tiktoken.get_encoding(config.name)
        except ValueError:
            self.enc = tiktoken.encoding_for_model(config.name)

    def encode(self, text: str) -> list[int]:
        ids = self.enc.encode_ordinary(text)
        if self.config.add_bos:
            ids = [self.enc.eot_token] + ids
        if self.config.add_eos:
            ids = ids + [self.enc.eot_token]
        return ids

    def decode(self, ids: list[int]) -> str:
        return self.enc.decode(list(ids))

    @property
    def vocab_size(self) -> int:
        return self.enc.n_vocab

    @property
    def eos_token_id(self) -> int:
        return self.enc.eot_token

    @property
    def bos_token_id(self) -> int:
        return self.enc.eot_token
