"""OLMo-3 family (optimus_dl/modules/model/olmo3.py:49-399): post-norm residual blocks
``x + norm(attn(x))``, ``x + norm(mlp(x))``; per-layer ``sliding_attention`` / ``full_attention``;
QK-norm over the full q / k width (not per head); ``rope_parameters`` dict (YaRN capable)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from ..ops.rope import precompute_freqs_cis
from . import register_model
from .blocks.attention import RotarySelfAttention
from .blocks.layer_norms import RMSNorm
from .blocks.mlp import SwiGLUMLP
from .gpt2 import GPTConfig
from .llama2 import Llama


@dataclass
class Olmo3Config(GPTConfig):
    sequence_length: int = 4096
    rmsnorm_eps: float = 1e-6
    rope_theta: float = 500000.0
    rope_parameters: dict = field(default_factory=lambda: {"rope_type": "default"})
    head_dim: int | None = None
    bias: bool = False
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    n_kv_head: int | None = 4
    intermediate_size: int | None = 1024
    multiple_of: int = 256
    sliding_window: int = 4096
    n_layer: int = 16
    layer_types: list[str] = field(default_factory=lambda: (["sliding_attention"] * 3 + ["full_attention"]) * 4)
    use_liger_rmsnorm: bool | None = None
    use_liger_swiglu: bool | None = None


class Olmo3Attention(RotarySelfAttention):
    def __init__(self, config, layer_idx: int):
        self.layer_type = config.layer_types[layer_idx]
        self.layer_idx = layer_idx
        assert self.layer_type in ("sliding_attention", "full_attention")
        window = config.sliding_window if self.layer_type == "sliding_attention" else None
        super().__init__(n_embd=config.n_embd, n_head=config.n_head, n_kv_head=config.n_kv_head,
                         head_dim=config.head_dim, dropout=config.dropout, bias=config.attention_bias,
                         use_qk_norm=True, qk_norm_per_head=False, rmsnorm_eps=config.rmsnorm_eps,
                         sliding_window=window)


class Olmo3Block(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.attn = Olmo3Attention(config, layer_idx)
        self.post_attention_layernorm = RMSNorm(config.n_embd, eps=config.rmsnorm_eps)
        self.mlp = SwiGLUMLP(n_embd=config.n_embd, intermediate_size=config.intermediate_size,
                             multiple_of=config.multiple_of, bias=False)
        self.post_feedforward_layernorm = RMSNorm(config.n_embd, eps=config.rmsnorm_eps)

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        x = x + self.post_attention_layernorm(self.attn(x, **kw))
        return x + self.post_feedforward_layernorm(self.mlp(x))


@register_model("olmo3", Olmo3Config)
class Olmo3(Llama):
    def __init__(self, config, **_):
        assert config.n_layer == len(config.layer_types), "Number of layers must match the length of layer_types"
        super().__init__(config)

    def _make_freqs(self, config) -> torch.Tensor:
        params = dict(config.rope_parameters)
        theta = params.get("rope_theta", config.rope_theta)
        return precompute_freqs_cis(self._head_dim(config), config.sequence_length, theta=theta, scaling_config=params)

    def _build_transformer(self, config) -> dict:
        return dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd, padding_idx=config.padding_token_id),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([Olmo3Block(config, i) for i in range(config.n_layer)]),
            ln_f=RMSNorm(config.n_embd, eps=config.rmsnorm_eps),
        )
