"""Tokenizer interface (optimus_dl/modules/tokenizer/base.py:12-76)."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any


class BaseTokenizer(ABC):
    def __init__(self, config: Any):
        self.config = config

    @abstractmethod
    def encode(self, text: str) -> list[int]: ...

    @abstractmethod
    def decode(self, ids: list[int]) -> str: ...

    @property
    @abstractmethod
    def vocab_size(self) -> int: ...

    @property
    def bos_token_id(self) -> int | None:
        return None

    @property
    def eos_token_id(self) -> int | None:
        return None

    def save_pretrained(self, save_directory: str) -> None:
        raise NotImplementedError(f"{type(self).__name__} cannot be saved in the Hugging Face layout")

    def apply_chat_template(self, conversation: list[dict[str, str]], tokenize: bool = True,
                            add_generation_prompt: bool = True, **kwargs: Any) -> Any:
        """Default template: ``role: content`` lines, then ``assistant:`` when a reply is expected."""
        text = "".join(f"{m['role']}: {m['content']}\n" for m in conversation)
        if add_generation_prompt:
            text += "assistant:"
        return self.encode(text) if tokenize else text
