"""Tokenizer config base (optimus_dl/modules/tokenizer/config.py)."""

from __future__ import annotations

from dataclasses import dataclass

from ..core.registry import RegistryConfig


@dataclass
class BaseTokenizerConfig(RegistryConfig):
    add_bos: bool = True
    add_eos: bool = True
