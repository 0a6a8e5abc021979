"""``transformers``: wraps ``AutoTokenizer`` incl. chat templates
(optimus_dl/modules/tokenizer/implementations/huggingface.py)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .. import register_tokenizer
from ..base import BaseTokenizer
from ..config import BaseTokenizerConfig


@dataclass
class HFTokenizerConfig(BaseTokenizerConfig):
    name: str = "gpt2"
    trust_remote_code: bool = False
    tokenizer_kwargs: dict = field(default_factory=dict)


@register_tokenizer("transformers", HFTokenizerConfig)
class HFTokenizer(BaseTokenizer):
    def __init__(self, config, **kwargs: Any):
        super().__init__(config)
        from transformers import AutoTokenizer

        self.tokenizer = AutoTokenizer.from_pretrained(config.name, trust_remote_code=bool(config.trust_remote_code),
                                                       **dict(config.get("tokenizer_kwargs") or {}))

    def encode(self, text: str) -> list[int]:
        ids = self.tokenizer.encode(text, add_special_tokens=False)
        if self.config.add_bos and self.bos_token_id is not None:
            ids = [self.bos_token_id] + ids
        if self.config.add_eos and self.eos_token_id is not None:
            ids = ids + [self.eos_token_id]
        return ids

    def decode(self, ids: list[int]) -> str:
        return self.tokenizer.decode(ids)

    @property
    def vocab_size(self) -> int:
        return len(self.tokenizer)

    @property
    def bos_token_id(self) -> int | None:
        return self.tokenizer.bos_token_id

    @property
    def eos_token_id(self) -> int | None:
        return self.tokenizer.eos_token_id

    def save_pretrained(self, save_directory: str) -> None:
        self.tokenizer.save_pretrained(save_directory)

    def apply_chat_template(self, conversation, tokenize: bool = True, add_generation_prompt: bool = True, **kwargs: Any):
        if getattr(self.tokenizer, "chat_template", None):
            return self.tokenizer.apply_chat_template(conversation, tokenize=tokenize,
                                                      add_generation_prompt=add_generation_prompt, **kwargs)
        return super().apply_chat_template(conversation, tokenize, add_generation_prompt, **kwargs)
