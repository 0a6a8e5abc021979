"""Causal self-attention with document masks, sliding windows and GQA.

One entry point, :func:`qkv_attention`, covers every masking mode of the reference's
attention block (optimus_dl/modules/model/blocks/attention.py:44-65,359-521): plain causal,
packed variable-length batches (``cu_seqlens``), per-token ``document_ids``, padded batches
(``seq_lens``) and left sliding windows. All of them reduce to one description that the
kernels consume: tokens are laid out as one flat stream of ``B*T`` positions and every query
``i`` may attend keys ``j`` with ``lo[i] <= j <= i`` where
``lo[i] = max(doc_start[i], i - window + 1)`` and ``doc_start[i]`` is the flat index of the first
token of ``i``'s document (or sequence).

On CUDA bf16 the hand-written tcgen05 kernels in ``csrc/attention.cu`` run; QK-norm and RoPE are
applied by ``csrc/rope.cu`` on the fused QKV projection output and the backward writes dq, dk, dv
straight into one ``d(qkv)`` buffer. Elsewhere a PyTorch reference (explicit mask + SDPA math)
runs; it is also the oracle for the kernel tests.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import _lib, rope as rope_ops
from .norm import rms_norm_ref


class BoundaryError(ValueError, AssertionError):
    """Document boundaries that do not cover the batch exactly."""


def build_doc_start(B: int, T: int, device: torch.device, document_ids: torch.Tensor | None = None,
                    cu_seqlens: torch.Tensor | None = None) -> torch.Tensor:
    """Flat ``int32 [B*T]`` index of the first token of each token's document."""
    idx = torch.arange(B * T, device=device, dtype=torch.int64).view(B, T)
    if cu_seqlens is not None:
        if not cu_seqlens.is_cuda and cu_seqlens.numel() > 0:
            # host-side boundaries can be checked without a device synchronisation: they must cover the batch exactly
            # (same two conditions and wording as optimus_dl/modules/model/blocks/attention.py:282-287)
            if int(cu_seqlens[0]) != 0:
                raise BoundaryError(f"cu_seqlens must start with 0, got {int(cu_seqlens[0])}")
            if int(cu_seqlens[-1]) != B * T:
                raise BoundaryError(f"cu_seqlens[-1] ({int(cu_seqlens[-1])}) must match sequence length T ({B * T})")
        cu = cu_seqlens.to(device=device, dtype=torch.int64)
        flat = idx.view(-1)
        seg = torch.searchsorted(cu, flat, right=True) - 1
        start = cu[seg.clamp(min=0, max=cu.numel() - 1)]
        # tokens past the last boundary (padding) start their own segment at the last boundary
        return start.to(torch.int32)
    if document_ids is not None:
        d = document_ids.to(device)
        new_run = torch.ones((B, T), dtype=torch.bool, device=device)
        new_run[:, 1:] = d[:, 1:] != d[:, :-1]
        start = torch.where(new_run, idx, torch.zeros_like(idx))
        start = torch.cummax(start, dim=1).values
        return start.view(-1).to(torch.int32)
    return (idx // T * T).view(-1).to(torch.int32)


def mask_from_doc_start(doc_start: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """Dense boolean ``[N, N]`` mask (True = attend) equivalent to the kernel's rule."""
    N = doc_start.numel()
    i = torch.arange(N, device=doc_start.device)
    lo = doc_start.to(torch.int64)
    if window is not None and window > 0:
        lo = torch.maximum(lo, i - window + 1)
    j = i.view(1, N)
    return (j <= i.view(N, 1)) & (j >= lo.view(N, 1))


def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, doc_start: torch.Tensor,
                  window: int | None = None, scale: float | None = None) -> torch.Tensor:
    """fp32 reference. ``q [N, Hq, hd]``, ``k, v [N, Hk, hd]`` over the flat token stream."""
    N, Hq, hd = q.shape
    Hk = k.shape[1]
    rep = Hq // Hk
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    mask = mask_from_doc_start(doc_start, window)
    qf = q.float().transpose(0, 1)
    kf = k.float().repeat_interleave(rep, dim=1).transpose(0, 1)
    vf = v.float().repeat_interleave(rep, dim=1).transpose(0, 1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).transpose(0, 1).to(q.dtype)


def _kernel_ok(qkv: torch.Tensor, hd: int) -> bool:
    return qkv.is_cuda and qkv.dtype == torch.bfloat16 and hd in (64, 128) and hasattr(_lib.lib(), "ob_attn_fwd")


class _QKVAttention(torch.autograd.Function):
    """qkv [N, (Hq+2Hk)*hd] -> out [N, Hq*hd], all on the kernels."""

    @staticmethod
    def forward(ctx, qkv, freqs, pos_ids, qw, kw, doc_start, Hq, Hk, hd, window, eps, seq_len, scale):
        l = _lib.lib()
        N = qkv.shape[0]
        W = (Hq + 2 * Hk) * hd
        assert qkv.shape[1] == W and qkv.stride(1) == 1
        has_norm = qw is not None
        dev = qkv.device
        qw_b = qw.to(torch.bfloat16).contiguous() if has_norm else None
        kw_b = kw.to(torch.bfloat16).contiguous() if has_norm else None
        rstd = torch.empty((N, Hq + Hk), dtype=torch.float32, device=dev) if has_norm else None
        if freqs is not None or has_norm:
            if has_norm:
                # keep the pre-norm projections for the backward; rotate into a fresh buffer
                work = torch.empty_like(qkv)
                work[:, (Hq + Hk) * hd:].copy_(qkv[:, (Hq + Hk) * hd:])
            else:
                work = qkv  # rotation is its own inverse up to sign: rotate in place
            fr = freqs if freqs is not None else _identity_freqs(seq_len, hd, dev)
            rope_ops.rope_kernel_fwd(qkv, work, qkv.stride(0), work.stride(0), fr, pos_ids, qw_b, kw_b, rstd, N, Hq, Hk,
                                     hd, seq_len, eps)
        else:
            work = qkv
        out = torch.empty((N, Hq * hd), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((Hq, N), dtype=torch.float32, device=dev)
        q_ptr = work
        k_ptr = work[:, Hq * hd:]
        v_ptr = work[:, (Hq + Hk) * hd:]
        rc = l.ob_attn_fwd(_lib.ptr(q_ptr), _lib.ptr(k_ptr), _lib.ptr(v_ptr), _lib.ptr(out), _lib.ptr(lse),
                           _lib.ptr(doc_start), N, Hq, Hk, hd, work.stride(0), work.stride(0), out.stride(0),
                           float(scale), int(window or 0), _lib.ptr(_lib.status_word(dev)), _lib.stream())
        _lib.check(rc, "ob_attn_fwd")
        ctx.save_for_backward(work, out, lse, doc_start, freqs, pos_ids, qw_b, kw_b, rstd, qkv if has_norm else None)
        ctx.meta = (Hq, Hk, hd, window, seq_len, scale, has_norm, None if qw is None else qw.dtype)
        # note: without QK-norm the rotation overwrote ``qkv`` in place; the projection that
        # produced it does not need its output for its own backward, and callers treat it as consumed.
        return out

    @staticmethod
    def backward(ctx, dout):
        work, out, lse, doc_start, freqs, pos_ids, qw_b, kw_b, rstd, qkv_pre = ctx.saved_tensors
        Hq, Hk, hd, window, seq_len, scale, has_norm, wdtype = ctx.meta
        l = _lib.lib()
        N = work.shape[0]
        dev = work.device
        dout = dout.contiguous()
        dqkv = torch.empty_like(work)
        delta = torch.empty((Hq, N), dtype=torch.float32, device=dev)
        kv_last = torch.empty(((N + 127) // 128,), dtype=torch.int32, device=dev)
        rc = l.ob_attn_bwd(_lib.ptr(work), _lib.ptr(work[:, Hq * hd:]), _lib.ptr(work[:, (Hq + Hk) * hd:]),
                           _lib.ptr(out), _lib.ptr(dout), _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(dqkv),
                           _lib.ptr(dqkv[:, Hq * hd:]), _lib.ptr(dqkv[:, (Hq + Hk) * hd:]), _lib.ptr(doc_start),
                           _lib.ptr(kv_last), N, Hq, Hk, hd, work.stride(0), out.stride(0), dqkv.stride(0),
                           float(scale), int(window or 0), _lib.ptr(_lib.status_word(dev)), _lib.stream())
        _lib.check(rc, "ob_attn_bwd")
        dqw = dkw = None
        if freqs is not None or has_norm:
            fr = freqs if freqs is not None else _identity_freqs(seq_len, hd, dev)
            partial = None
            if has_norm:
                grid = rope_ops.rope_grid(N * (Hq + Hk))
                partial = torch.empty((grid, 2, hd), dtype=torch.float32, device=dev)
            rope_ops.rope_kernel_bwd(dqkv, dqkv, dqkv.stride(0), dqkv.stride(0), qkv_pre,
                                     qkv_pre.stride(0) if qkv_pre is not None else 0, fr, pos_ids, qw_b, kw_b, rstd,
                                     partial, N, Hq, Hk, hd, seq_len)
            if has_norm:
                s = partial.sum(0)
                dqw, dkw = s[0].to(wdtype), s[1].to(wdtype)
        return dqkv, None, None, dqw, dkw, None, None, None, None, None, None, None, None


_ident_cache: dict = {}


def _identity_freqs(seq_len: int, hd: int, device: torch.device) -> torch.Tensor:
    key = (seq_len, hd, str(device))
    if key not in _ident_cache:
        f = torch.zeros((max(seq_len, 1), hd // 2, 2), dtype=torch.float32, device=device)
        f[..., 0] = 1.0
        _ident_cache[key] = f
    return _ident_cache[key]


def qkv_attention(qkv: torch.Tensor, *, n_head: int, n_kv_head: int, head_dim: int, doc_start: torch.Tensor,
                  freqs_cis: torch.Tensor | None = None, position_ids: torch.Tensor | None = None,
                  q_norm_weight: torch.Tensor | None = None, k_norm_weight: torch.Tensor | None = None,
                  norm_eps: float = 1e-6, window: int | None = None, seq_len: int | None = None,
                  scale: float | None = None, dropout_p: float = 0.0) -> torch.Tensor:
    """Attention on a fused projection ``qkv [B, T, (Hq + 2 Hk) * hd]``; returns ``[B, T, Hq * hd]``.

    Order of operations matches the reference: per-head QK-norm (when weights are given), then
    interleaved RoPE (when ``freqs_cis`` is given), then masked softmax attention. ``dropout_p > 0``
    (dropout on the attention probabilities, optimus_dl/modules/model/blocks/attention.py:133, used by
    GPT-2 configurations that train with dropout) has no kernel of its own and takes the row-wise
    PyTorch path with its ``[B, T, T]`` mask.
    """
    B, T, W = qkv.shape
    Hq, Hk, hd = n_head, n_kv_head, head_dim
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    seq_len = seq_len or T
    if _kernel_ok(qkv, hd) and dropout_p == 0.0:
        pos = position_ids.reshape(-1).to(torch.int32).contiguous() if position_ids is not None else None
        fr = freqs_cis.to(device=qkv.device, dtype=torch.float32).contiguous() if freqs_cis is not None else None
        flat = qkv.reshape(B * T, W)
        out = _QKVAttention.apply(flat, fr, pos, q_norm_weight, k_norm_weight, doc_start, Hq, Hk, hd, window, norm_eps,
                                  seq_len, scale)
        return out.view(B, T, Hq * hd)
    q, k, v = qkv.split([Hq * hd, Hk * hd, Hk * hd], dim=-1)
    q = q.reshape(B, T, Hq, hd)
    k = k.reshape(B, T, Hk, hd)
    v = v.reshape(B, T, Hk, hd)
    if q_norm_weight is not None:
        q = rms_norm_ref(q, q_norm_weight, norm_eps)
        k = rms_norm_ref(k, k_norm_weight, norm_eps)
    if freqs_cis is not None:
        q, k = rope_ops.apply_rotary_emb(q, k, freqs_cis, position_ids)
    if dropout_p > 0.0:
        return attention_sdpa_rows(q, k, v, doc_start, window, scale, dropout_p).reshape(B, T, Hq * hd)
    out = attention_sdpa(q.reshape(B * T, Hq, hd), k.reshape(B * T, Hk, hd), v.reshape(B * T, Hk, hd), doc_start, window,
                         scale)
    return out.reshape(B, T, Hq * hd)


def attention_sdpa_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, doc_start: torch.Tensor, window: int | None,
                        scale: float, dropout_p: float = 0.0) -> torch.Tensor:
    """Differentiable PyTorch path per batch row: ``q [B, T, Hq, hd]``, ``k, v [B, T, Hk, hd]``, mask ``[B, 1, T, T]``
    built from the flat ``doc_start`` (a document never crosses a row), dropout on the probabilities."""
    B, T, Hq, hd = q.shape
    Hk = k.shape[2]
    i = torch.arange(T, device=q.device)
    lo = doc_start.to(torch.int64).view(B, T) - (torch.arange(B, device=q.device) * T).view(B, 1)
    if window is not None and window > 0:
        lo = torch.maximum(lo, (i - window + 1).view(1, T))
    j = i.view(1, 1, T)
    mask = ((j <= i.view(1, T, 1)) & (j >= lo.view(B, T, 1))).unsqueeze(1)
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if Hk != Hq:
        kh = kh.repeat_interleave(Hq // Hk, dim=1)
        vh = vh.repeat_interleave(Hq // Hk, dim=1)
    o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, dropout_p=dropout_p, scale=scale)
    return o.transpose(1, 2)


def attention_sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, doc_start: torch.Tensor,
                   window: int | None, scale: float) -> torch.Tensor:
    """Differentiable PyTorch path over the flat stream (explicit mask + SDPA)."""
    N, Hq, hd = q.shape
    Hk = k.shape[1]
    mask = mask_from_doc_start(doc_start, window)
    qh = q.transpose(0, 1).unsqueeze(0)
    kh = k.transpose(0, 1).unsqueeze(0)
    vh = v.transpose(0, 1).unsqueeze(0)
    if Hk != Hq:
        kh = kh.repeat_interleave(Hq // Hk, dim=1)
        vh = vh.repeat_interleave(Hq // Hk, dim=1)
    o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask, scale=scale)
    return o.squeeze(0).transpose(0, 1)


# ---------------------------------------------------------------------- inference helpers (no autograd)
@torch.no_grad()
def rotate_qkv(qkv: torch.Tensor, *, n_head: int, n_kv_head: int, head_dim: int,
               freqs_cis: torch.Tensor | None = None, position_ids: torch.Tensor | None = None,
               q_norm_weight: torch.Tensor | None = None, k_norm_weight: torch.Tensor | None = None,
               norm_eps: float = 1e-6, seq_len: int | None = None) -> torch.Tensor:
    """Per-head QK-norm and RoPE on a fused projection ``[B, T, (Hq + 2 Hk) * hd]``; returns the same layout."""
    B, T, W = qkv.shape
    Hq, Hk, hd = n_head, n_kv_head, head_dim
    has_norm = q_norm_weight is not None
    if freqs_cis is None and not has_norm:
        return qkv
    if _kernel_ok(qkv, hd):
        flat = qkv.reshape(B * T, W)
        pos = position_ids.reshape(-1).to(torch.int32).contiguous() if position_ids is not None else None
        fr = (freqs_cis.to(device=qkv.device, dtype=torch.float32).contiguous() if freqs_cis is not None
              else _identity_freqs(seq_len or T, hd, qkv.device))
        work = flat
        if has_norm:
            work = torch.empty_like(flat)
            work[:, (Hq + Hk) * hd:].copy_(flat[:, (Hq + Hk) * hd:])
        qw = q_norm_weight.to(torch.bfloat16).contiguous() if has_norm else None
        kw = k_norm_weight.to(torch.bfloat16).contiguous() if has_norm else None
        rstd = torch.empty((B * T, Hq + Hk), dtype=torch.float32, device=qkv.device) if has_norm else None
        rope_ops.rope_kernel_fwd(flat, work, flat.stride(0), work.stride(0), fr, pos, qw, kw, rstd, B * T, Hq, Hk, hd,
                                 seq_len or T, norm_eps)
        return work.view(B, T, W)
    q, k, v = qkv.split([Hq * hd, Hk * hd, Hk * hd], dim=-1)
    q = q.reshape(B, T, Hq, hd)
    k = k.reshape(B, T, Hk, hd)
    if has_norm:
        q = rms_norm_ref(q, q_norm_weight, norm_eps)
        k = rms_norm_ref(k, k_norm_weight, norm_eps)
    if freqs_cis is not None:
        q, k = rope_ops.apply_rotary_emb(q, k, freqs_cis, position_ids)
    return torch.cat([q.reshape(B, T, -1).to(qkv.dtype), k.reshape(B, T, -1).to(qkv.dtype), v], dim=-1)


@torch.no_grad()
def attention_rotated(work: torch.Tensor, *, n_head: int, n_kv_head: int, head_dim: int, doc_start: torch.Tensor,
                      window: int | None = None, scale: float | None = None) -> torch.Tensor:
    """Masked attention on an already normalised / rotated fused projection (prefill path)."""
    B, T, W = work.shape
    Hq, Hk, hd = n_head, n_kv_head, head_dim
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if _kernel_ok(work, hd):
        flat = work.reshape(B * T, W)
        N = B * T
        out = torch.empty((N, Hq * hd), dtype=torch.bfloat16, device=work.device)
        lse = torch.empty((Hq, N), dtype=torch.float32, device=work.device)
        rc = _lib.lib().ob_attn_fwd(_lib.ptr(flat), _lib.ptr(flat[:, Hq * hd:]), _lib.ptr(flat[:, (Hq + Hk) * hd:]),
                                    _lib.ptr(out), _lib.ptr(lse), _lib.ptr(doc_start), N, Hq, Hk, hd, flat.stride(0),
                                    flat.stride(0), out.stride(0), float(scale), int(window or 0),
                                    _lib.ptr(_lib.status_word(work.device)), _lib.stream())
        _lib.check(rc, "ob_attn_fwd")
        return out.view(B, T, Hq * hd)
    q, k, v = work.split([Hq * hd, Hk * hd, Hk * hd], dim=-1)
    out = attention_sdpa(q.reshape(B * T, Hq, hd), k.reshape(B * T, Hk, hd), v.reshape(B * T, Hk, hd), doc_start, window,
                         scale)
    return out.reshape(B, T, Hq * hd)
