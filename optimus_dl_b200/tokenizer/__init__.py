"""Tokenizers and the ``tokenizer`` registry (``_name``: char_tokenize, transformers, tiktoken,
inline_tokens_tokenizer)."""

from ..core.bootstrap import bootstrap_module
from ..core.registry import make_registry
from .base import BaseTokenizer
from .config import BaseTokenizerConfig

_TOKENIZER_REGISTRY, register_tokenizer, build_tokenizer = make_registry("tokenizer", BaseTokenizer)
bootstrap_module(__name__)
