"""Self-attention blocks (optimus_dl/modules/model/blocks/attention.py:68-612).

Same parameters (``wq, wk, wv, wo`` and optional ``q_norm, k_norm``) and the same forward
signature; the computation is one fused QKV projection, QK-norm + RoPE and masked attention in
``ops.attention.qkv_attention``, then the output projection. Full-width QK-norm (OLMo-3 style,
``qk_norm_per_head=False``) normalises the q and k slices before the per-head path.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import attention as attn_ops
from ...ops import linear as lin_ops
from .layer_norms import RMSNorm

# Which attention back ends exist, under the names of optimus_dl/modules/model/blocks/attention.py:24-40. The
# reference picks flash-attn / flex attention / SDPA by these flags; here every masked form (causal, sliding
# window, packed documents, per-row lengths) runs in the same kernels, so both are true wherever those kernels
# are, and code that switches them off only loses nothing.
FLASH_ATTENTION_AVAILABLE = True
FLEX_ATTENTION_AVAILABLE = True


def attention_mask_fn(b, _, q_idx, kv_idx, window_size=None, seq_lens=None, document_ids=None):
    """The visibility rule of every attention path, as a predicate over index tensors (same arguments as
    optimus_dl/modules/model/blocks/attention.py:44-65): key ``kv_idx`` is visible to query ``q_idx`` of sample ``b``
    when it is not in the future, lies inside the sliding window, both positions are inside the sample's length,
    and both belong to the same document. The kernels do not evaluate this function; they derive the same set from
    one ``doc_start`` index per token (``ops.attention.build_doc_start``), and tests compare the two."""
    visible = kv_idx <= q_idx
    if window_size is not None:
        visible = visible & (q_idx - kv_idx < window_size)
    if seq_lens is not None:
        visible = visible & (q_idx < seq_lens[b]) & (kv_idx < seq_lens[b])
    if document_ids is not None:
        visible = visible & (document_ids[b, q_idx] == document_ids[b, kv_idx])
    return visible


class BaseSelfAttention(nn.Module):
    use_rope = False

    def __init__(self, n_embd: int, n_head: int, n_kv_head: int | None = None, head_dim: int | None = None,
                 dropout: float = 0.0, bias: bool = False, use_qk_norm: bool = False, qk_norm_per_head: bool = True,
                 rmsnorm_eps: float = 1e-5, sliding_window: int | None = None):
        super().__init__()
        assert n_embd % n_head == 0, "n_embd must be divisible by n_head"
        self.n_head = n_head
        self.n_kv_head = n_kv_head if n_kv_head is not None else n_head
        assert self.n_head % self.n_kv_head == 0, "n_head must be divisible by n_kv_head"
        self.n_rep = self.n_head // self.n_kv_head
        self.head_dim = head_dim or n_embd // n_head
        self.n_embd = n_embd
        self.dropout = dropout
        self.use_qk_norm = use_qk_norm
        self.qk_norm_per_head = qk_norm_per_head
        self.sliding_window = sliding_window
        self.rmsnorm_eps = rmsnorm_eps
        self.wq = nn.Linear(n_embd, n_head * self.head_dim, bias=bias)
        self.wk = nn.Linear(n_embd, self.n_kv_head * self.head_dim, bias=bias)
        self.wv = nn.Linear(n_embd, self.n_kv_head * self.head_dim, bias=bias)
        self.wo = nn.Linear(n_head * self.head_dim, n_embd, bias=bias)
        if use_qk_norm:
            qd = self.head_dim if qk_norm_per_head else n_head * self.head_dim
            kd = self.head_dim if qk_norm_per_head else self.n_kv_head * self.head_dim
            self.q_norm = RMSNorm(qd, eps=rmsnorm_eps)
            self.k_norm = RMSNorm(kd, eps=rmsnorm_eps)
        self.attn_dropout = nn.Dropout(dropout)      # holds the rate; applied inside the attention product
        self.resid_dropout = nn.Dropout(dropout)
        # tensor-parallel state (parallel.tp.TPState), set by apply_tensor_parallel together with local head counts
        self.tp = None
        # decoding state (recipe.generation.LayerKV) while a generation session is active
        self.kv = None

    def forward(self, x: torch.Tensor, freqs_cis: torch.Tensor | None = None, seq_lens: torch.Tensor | None = None,
                document_ids: torch.Tensor | None = None, position_ids: torch.Tensor | None = None,
                cu_seqlens: torch.Tensor | None = None, max_seqlen: int | None = None,
                doc_start: torch.Tensor | None = None) -> torch.Tensor:
        if self.kv is not None:
            return self._forward_cached(x, freqs_cis, position_ids)
        if self.tp is not None:
            from ...parallel import tp as tp_ops

            B, T = self.tp.full_shape
            if doc_start is None:
                doc_start = attn_ops.build_doc_start(B, T, x.device, document_ids, cu_seqlens)
            return tp_ops.attention_forward(self, x, freqs_cis=freqs_cis, position_ids=position_ids,
                                            doc_start=doc_start)
        B, T, _ = x.shape
        if cu_seqlens is not None:
            assert B == 1, f"cu_seqlens is only supported for flat batches (B=1), but got B={B}"
            assert cu_seqlens.ndim == 1, f"cu_seqlens must be a 1D tensor, got ndim={cu_seqlens.ndim}"
        if doc_start is None:
            doc_start = attn_ops.build_doc_start(B, T, x.device, document_ids, cu_seqlens)
        biases = [self.wq.bias, self.wk.bias, self.wv.bias]
        qkv = lin_ops.multi_linear(x, [self.wq.weight, self.wk.weight, self.wv.weight], biases)
        Hq, Hk, hd = self.n_head, self.n_kv_head, self.head_dim
        qw = kw = None
        if self.use_qk_norm:
            if self.qk_norm_per_head:
                qw, kw = self.q_norm.weight, self.k_norm.weight
            else:
                q, k, v = qkv.split([Hq * hd, Hk * hd, Hk * hd], dim=-1)
                qkv = torch.cat([self.q_norm(q.contiguous()), self.k_norm(k.contiguous()), v], dim=-1)
        y = attn_ops.qkv_attention(qkv, n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=doc_start,
                                   freqs_cis=freqs_cis if self.use_rope else None,
                                   position_ids=position_ids if self.use_rope else None, q_norm_weight=qw,
                                   k_norm_weight=kw, norm_eps=self.rmsnorm_eps, window=self.sliding_window,
                                   dropout_p=self.attn_dropout.p if self.training else 0.0)
        y = lin_ops.linear(y, self.wo.weight, self.wo.bias)
        return self.resid_dropout(y) if self.training and self.resid_dropout.p > 0 else y


    @torch.no_grad()
    def _forward_cached(self, x: torch.Tensor, freqs_cis: torch.Tensor | None, position_ids: torch.Tensor | None):
        """Inference with a key/value cache: a multi-token call is a prefill that fills the cache, a
        one-token call attends over the cache with the decode kernel (which also appends)."""
        from ...ops import decode as dec_ops

        kv = self.kv
        B, T, _ = x.shape
        Hq, Hk, hd = self.n_head, self.n_kv_head, self.head_dim
        qkv = lin_ops.multi_linear(x, [self.wq.weight, self.wk.weight, self.wv.weight],
                                   [self.wq.bias, self.wk.bias, self.wv.bias])
        qw = kw = None
        if self.use_qk_norm:
            if self.qk_norm_per_head:
                qw, kw = self.q_norm.weight, self.k_norm.weight
            else:
                q, k, v = qkv.split([Hq * hd, Hk * hd, Hk * hd], dim=-1)
                qkv = torch.cat([self.q_norm(q.contiguous()), self.k_norm(k.contiguous()), v], dim=-1)
        if position_ids is None:
            position_ids = (kv.seq_lens.to(torch.long)[:, None] - T
                            + torch.arange(T, device=x.device)[None, :]) if kv.filled else None
        work = attn_ops.rotate_qkv(qkv.contiguous(), n_head=Hq, n_kv_head=Hk, head_dim=hd,
                                   freqs_cis=freqs_cis if self.use_rope else None,
                                   position_ids=position_ids if self.use_rope else None, q_norm_weight=qw,
                                   k_norm_weight=kw, norm_eps=self.rmsnorm_eps)
        k_new = work[..., Hq * hd:(Hq + Hk) * hd].reshape(B, T, Hk, hd)
        v_new = work[..., (Hq + Hk) * hd:].reshape(B, T, Hk, hd)
        if T > 1 or not kv.filled:
            assert not kv.filled, "multi-token calls are only supported as the prefill of an empty cache"
            kv.k[:, :T].copy_(k_new)
            kv.v[:, :T].copy_(v_new)
            doc_start = attn_ops.build_doc_start(B, T, x.device, None, None)
            y = attn_ops.attention_rotated(work, n_head=Hq, n_kv_head=Hk, head_dim=hd, doc_start=doc_start,
                                           window=self.sliding_window)
        else:
            w2 = work.view(B, -1)
            q = w2[:, : Hq * hd].unflatten(1, (Hq, hd))
            kn = w2[:, Hq * hd:(Hq + Hk) * hd].unflatten(1, (Hk, hd))
            vn = w2[:, (Hq + Hk) * hd:].unflatten(1, (Hk, hd))
            y = dec_ops.decode_attention(q, kn, vn, kv.k, kv.v, kv.seq_lens, window=self.sliding_window,
                                         n_splits=kv.n_splits, workspace=kv.workspace).view(B, 1, Hq * hd)
        return lin_ops.linear(y, self.wo.weight, self.wo.bias)


class CausalSelfAttention(BaseSelfAttention):
    """GPT-2 attention: built from a config with ``n_embd, n_head, dropout, bias`` and no RoPE."""

    def __init__(self, config):
        super().__init__(n_embd=config.n_embd, n_head=config.n_head, n_kv_head=None,
                         head_dim=getattr(config, "head_dim", None), dropout=config.dropout, bias=config.bias)


class RotarySelfAttention(BaseSelfAttention):
    use_rope = True
