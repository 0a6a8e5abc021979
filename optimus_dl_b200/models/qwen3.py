"""Qwen-3 family (optimus_dl/modules/model/qwen3.py:32-380): Llama layout with an explicit
``head_dim``, per-head RMSNorm on q and k before RoPE, optional sliding window, attention bias."""

from __future__ import annotations

from dataclasses import dataclass

from . import register_model
from .blocks.transformer import RotaryTransformerBlock
from .llama2 import Llama, LlamaConfig


@dataclass
class Qwen3Config(LlamaConfig):
    head_dim: int | None = None
    sliding_window: int | None = None
    attention_bias: bool = True
    rmsnorm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    sequence_length: int = 32768
    use_qk_norm: bool = True


class Qwen3Block(RotaryTransformerBlock):
    def __init__(self, config):
        super().__init__(n_embd=config.n_embd, n_head=config.n_head, n_kv_head=config.n_kv_head,
                         head_dim=config.head_dim, dropout=config.dropout, rmsnorm_eps=config.rmsnorm_eps,
                         bias=config.bias, attention_bias=config.attention_bias,
                         intermediate_size=config.intermediate_size, multiple_of=config.multiple_of, use_qk_norm=True,
                         qk_norm_per_head=True, mlp_type=config.mlp_type, sliding_window=config.sliding_window)


@register_model("qwen3", Qwen3Config)
class Qwen3(Llama):
    block_cls = Qwen3Block


@Qwen3.register_arch("0.6B")
def qwen3_0_6b():
    return Qwen3Config(n_layer=28, n_head=16, n_kv_head=8, n_embd=1024, head_dim=128, intermediate_size=3072,
                       vocab_size=151936, tie_word_embeddings=True, rope_theta=1000000.0, sequence_length=40960,
                       attention_bias=False)


@Qwen3.register_arch("4B")
def qwen3_4b():
    return Qwen3Config(n_layer=36, n_head=32, n_kv_head=8, n_embd=2560, intermediate_size=9216, multiple_of=256,
                       attention_bias=True)


@Qwen3.register_arch("1.7B")
def qwen3_1_7b():
    """Policy shape of the GRPO recipe."""
    return Qwen3Config(n_layer=28, n_head=16, n_kv_head=8, n_embd=2048, head_dim=128, intermediate_size=6144,
                       vocab_size=151936, tie_word_embeddings=True, attention_bias=False, sequence_length=4096)


@Qwen3.register_arch("14B")
def qwen3_14b():
    return Qwen3Config(n_layer=40, n_head=40, n_kv_head=8, n_embd=5120, head_dim=128, intermediate_size=17408,
                       vocab_size=151936, tie_word_embeddings=False, attention_bias=False, sequence_length=16384)
