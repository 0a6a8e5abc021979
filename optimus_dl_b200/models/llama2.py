"""Llama-2 / Llama-3 family (optimus_dl/modules/model/llama2.py:45-443): RMSNorm, rotary
attention with GQA, SwiGLU / ReLU^2 / GELU MLP, optional QK-norm, RoPE scaling, untied or tied
head. ``Llama3-8B`` is ``LlamaConfig(n_layer=32, n_embd=4096, n_head=32, n_kv_head=8,
intermediate_size=14336, vocab_size=128256, rope_theta=5e5, tie_word_embeddings=False)``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.nn as nn

from ..ops import attention as attn_ops
from ..ops.rope import precompute_freqs_cis
from . import register_model
from .blocks.layer_norms import RMSNorm
from .blocks.transformer import RotaryTransformerBlock
from .gpt2 import GPT, GPTConfig


@dataclass
class LlamaConfig(GPTConfig):
    sequence_length: int = 16000
    rmsnorm_eps: float = 1e-5
    bias: bool = False
    attention_bias: bool = False
    tie_word_embeddings: bool = True
    n_kv_head: int | None = None
    intermediate_size: int | None = None
    multiple_of: int = 256
    rope_theta: float = 10000.0
    rope_scaling: dict | None = None
    use_liger_rmsnorm: bool | None = None
    use_liger_swiglu: bool | None = None
    use_qk_norm: bool = False
    mlp_type: str = "swiglu"
    zero_init_projections: bool = False


class LlamaBlock(RotaryTransformerBlock):
    def __init__(self, config):
        super().__init__(n_embd=config.n_embd, n_head=config.n_head, n_kv_head=config.n_kv_head,
                         head_dim=getattr(config, "head_dim", None),
                         dropout=config.dropout, rmsnorm_eps=config.rmsnorm_eps, bias=config.bias,
                         attention_bias=config.attention_bias, intermediate_size=config.intermediate_size,
                         multiple_of=config.multiple_of, use_qk_norm=config.use_qk_norm, mlp_type=config.mlp_type)


@register_model("llama2", LlamaConfig)
class Llama(GPT):
    block_cls: Any = LlamaBlock

    def __init__(self, config, **_):
        self._freqs_cache: dict = {}
        super().__init__(config)
        if getattr(config, "zero_init_projections", False):
            # the feed-forward output projections start at zero; the attention output projection keeps its scaled
            # normal initialisation (optimus_dl/modules/model/llama2.py:196-213)
            for name, p in self.named_parameters():
                if name.endswith("c_proj.weight"):
                    nn.init.zeros_(p)
        self.head_dim = self._head_dim(config)
        self.freqs_cis = self._make_freqs(config)

    def _head_dim(self, config) -> int:
        return getattr(config, "head_dim", None) or config.n_embd // config.n_head

    def _make_freqs(self, config) -> torch.Tensor:
        return precompute_freqs_cis(self._head_dim(config), config.sequence_length, config.rope_theta,
                                    getattr(config, "rope_scaling", None))

    def _build_transformer(self, config) -> dict:
        return dict(
            wte=nn.Embedding(config.vocab_size, config.n_embd, padding_idx=config.padding_token_id),
            drop=nn.Dropout(config.dropout),
            h=nn.ModuleList([self.block_cls(config) for _ in range(config.n_layer)]),
            ln_f=RMSNorm(config.n_embd, eps=config.rmsnorm_eps),
        )

    def freqs_on(self, device: torch.device) -> torch.Tensor:
        """The cos/sin table on ``device`` (moved once and cached, not on every forward)."""
        key = str(device)
        f = self._freqs_cache.get(key)
        if f is None or f.shape != self.freqs_cis.shape:
            f = self.freqs_cis.to(device=device, dtype=torch.float32).contiguous()
            self._freqs_cache = {key: f}
        return f

    def block_kwargs(self, i: int, block: nn.Module, common: dict) -> dict:
        return common

    def forward(self, input_ids: torch.Tensor, seq_lens=None, document_ids=None, position_ids=None, cu_seqlens=None,
                max_seqlen=None, skip_lm_head: bool = False, **kwargs):
        B, T = input_ids.shape
        assert T <= self.config.sequence_length, f"sequence of length {T} exceeds {self.config.sequence_length}"
        tp = getattr(self, "_tp", None)
        if tp is not None:
            tp.full_shape = (B, T)
        x = self.transformer.drop(self.embed(input_ids))
        doc_start = attn_ops.build_doc_start(B, T, x.device, document_ids, cu_seqlens)
        common = dict(freqs_cis=self.freqs_on(x.device), seq_lens=seq_lens, document_ids=document_ids,
                      position_ids=position_ids, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, doc_start=doc_start)
        for i, block in enumerate(self.transformer.h):
            x = block(x, **self.block_kwargs(i, block, common))
        x = self.transformer.ln_f(x)
        if skip_lm_head:
            if tp is not None:
                from ..parallel import tp as tp_ops

                x = tp_ops.hidden_forward(self, x)
            return {"hidden": x}
        return {"logits": self.head(x)}

    def apply_tp(self, mesh, loss_parallel: bool = False, sequence_parallel: bool = False, **kwargs):
        """Shard the model over the tensor-parallel mesh (same options as the reference's ``apply_tp``)."""
        from ..parallel.tp import apply_tensor_parallel

        apply_tensor_parallel(self, mesh, loss_parallel=loss_parallel, sequence_parallel=sequence_parallel, **kwargs)


@Llama.register_arch("7b")
def llama_7b():
    return LlamaConfig(n_layer=32, n_head=32, n_embd=4096, multiple_of=256)


@Llama.register_arch("1b")
def llama_1b():
    return LlamaConfig(n_layer=18, n_head=32, n_embd=2048, multiple_of=4)


@Llama.register_arch("210M")
def llama_210m():
    return LlamaConfig(n_layer=24, n_head=12, n_embd=768, multiple_of=4)


@Llama.register_arch("lite")
def llama_lite():
    return LlamaConfig(n_layer=6, n_head=8, n_embd=768, multiple_of=4)


@Llama.register_arch("x-lite")
def llama_x_lite():
    return LlamaConfig(n_layer=6, n_head=4, n_embd=256, multiple_of=4)


@Llama.register_arch("3-8b")
def llama3_8b():
    """Llama-3-8B shape used by the flagship benchmark."""
    return LlamaConfig(n_layer=32, n_head=32, n_kv_head=8, n_embd=4096, intermediate_size=14336, vocab_size=128256,
                       rope_theta=500000.0, sequence_length=8192, tie_word_embeddings=False, rmsnorm_eps=1e-5)
