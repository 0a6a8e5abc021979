"""Pre-norm transformer block with rotary attention
(optimus_dl/modules/model/blocks/transformer.py:13-104): ``x + attn(ln_1(x))``, ``x + mlp(ln_2(x))``."""

from __future__ import annotations

import torch
import torch.nn as nn

from ...core.profile import nvtx_range
from .attention import RotarySelfAttention
from .layer_norms import RMSNorm
from .mlp import build_mlp


class RotaryTransformerBlock(nn.Module):
    def __init__(self, *, n_embd: int, n_head: int, n_kv_head: int | None = None, head_dim: int | None = None,
                 dropout: float = 0.0, rmsnorm_eps: float = 1e-5, bias: bool = False, attention_bias: bool = False,
                 intermediate_size: int | None = None, multiple_of: int = 256, use_qk_norm: bool = False,
                 qk_norm_per_head: bool = True, mlp_type: str = "swiglu", sliding_window: int | None = None,
                 use_liger_rmsnorm: bool | None = None, use_liger_swiglu: bool | None = None):
        super().__init__()
        self.ln_1 = RMSNorm(n_embd, eps=rmsnorm_eps)
        self.attn = RotarySelfAttention(n_embd=n_embd, n_head=n_head, n_kv_head=n_kv_head, head_dim=head_dim,
                                        dropout=dropout, bias=attention_bias, use_qk_norm=use_qk_norm,
                                        qk_norm_per_head=qk_norm_per_head, rmsnorm_eps=rmsnorm_eps,
                                        sliding_window=sliding_window)
        self.ln_2 = RMSNorm(n_embd, eps=rmsnorm_eps)
        self.mlp = build_mlp(mlp_type, n_embd, intermediate_size, multiple_of, bias, dropout)

    def forward(self, x: torch.Tensor, *, freqs_cis: torch.Tensor | None = None, seq_lens=None, document_ids=None,
                position_ids=None, cu_seqlens=None, max_seqlen=None, doc_start=None) -> torch.Tensor:
        with nvtx_range("block/attention"):
            a = self.attn(self.ln_1(x), freqs_cis=freqs_cis, seq_lens=seq_lens, document_ids=document_ids,
                          position_ids=position_ids, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, doc_start=doc_start)
        with nvtx_range("block/mlp"):
            # second norm fuses the residual add: h = x + a, y = norm(h)
            y, h = self.ln_2(a, residual=x)
            return self.mlp(y, residual=h)
