"""Inference-time ops: single-query attention over a KV cache and the fused token sampler.

The reference generates by re-running the whole prefix for every new token
(optimus_dl/modules/metrics/sources/generation.py:97-160, optimus_dl/recipe/serve/base.py); here
a decode step reads each cached key / value once (``csrc/attention_decode.cu``, which also appends
the new token's key / value to the cache) and picks the next token with one launch
(``csrc/sampler.cu``: temperature, top-k, top-p and the categorical draw without sorting).
Both have PyTorch fallbacks with the same semantics for CPU runs and tests.
"""

from __future__ import annotations

import math

import torch

from . import _lib


def _kernel_ok(*ts: torch.Tensor) -> bool:
    return all(t.is_cuda for t in ts) and _lib.available()


def decode_attention(q: torch.Tensor, k_new: torch.Tensor | None, v_new: torch.Tensor | None, k_cache: torch.Tensor,
                     v_cache: torch.Tensor, seq_lens: torch.Tensor, *, scale: float | None = None,
                     window: int | None = None, n_splits: int = 1, workspace: dict | None = None) -> torch.Tensor:
    """Attention of one query token per sequence against its cache.

    ``q``: ``[B, Hq, hd]`` (may be a strided view into a fused qkv row); ``k_new``/``v_new``:
    ``[B, Hk, hd]`` of the current token, stored at row ``seq_lens[b] - 1`` of the caches
    ``[B, Tmax, Hk, hd]`` (any batch / token / head strides; a head-major allocation viewed this way reads
    fastest) before attending (pass ``None`` if already stored); ``seq_lens``: int32
    ``[B]``, counts *including* the current token. Returns ``[B, Hq, hd]``.
    """
    B, Hq, hd = q.shape
    Tmax, Hk = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if (_kernel_ok(q, k_cache, v_cache) and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and hd in (64, 128) and Hq // Hk <= 8 and q.stride(2) == 1 and q.stride(1) == hd
            and k_cache.stride(3) == 1 and v_cache.stride() == k_cache.stride()):
        out = torch.empty((B, Hq, hd), dtype=torch.bfloat16, device=q.device)
        part_o = part_ml = None
        if n_splits > 1:
            ws = workspace if workspace is not None else {}
            key = (B, Hq, hd, n_splits)
            if ws.get("key") != key:
                ws["key"] = key
                ws["o"] = torch.empty(B * Hq * n_splits * hd, dtype=torch.float32, device=q.device)
                ws["ml"] = torch.empty(B * Hq * n_splits * 2, dtype=torch.float32, device=q.device)
            part_o, part_ml = ws["o"], ws["ml"]
        new_stride = 0
        if k_new is not None:
            assert k_new.stride(2) == 1 and k_new.stride(1) == hd and v_new.stride() == k_new.stride()
            new_stride = k_new.stride(0)
        rc = _lib.lib().ob_attn_decode(
            _lib.ptr(q), q.stride(0), _lib.ptr(k_new), _lib.ptr(v_new), new_stride, _lib.ptr(k_cache), _lib.ptr(v_cache),
            k_cache.stride(0), k_cache.stride(1), k_cache.stride(2), _lib.ptr(seq_lens), _lib.ptr(out), out.stride(0), _lib.ptr(part_o),
            _lib.ptr(part_ml), B, Hq, Hk, hd, int(n_splits), Tmax, float(scale), int(window or 0), _lib.stream())
        _lib.check(rc, "ob_attn_decode")
        return out
    return decode_attention_ref(q, k_new, v_new, k_cache, v_cache, seq_lens, scale=scale, window=window)


def decode_attention_ref(q, k_new, v_new, k_cache, v_cache, seq_lens, *, scale=None, window=None) -> torch.Tensor:
    """fp32 PyTorch statement of :func:`decode_attention` (also appends to the caches)."""
    B, Hq, hd = q.shape
    Tmax, Hk = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    lens = seq_lens.to(torch.long).clamp(0, Tmax)
    if k_new is not None:
        rows = torch.arange(B, device=q.device)
        ok = lens > 0
        k_cache[rows[ok], lens[ok] - 1] = k_new[ok].to(k_cache.dtype)
        v_cache[rows[ok], lens[ok] - 1] = v_new[ok].to(v_cache.dtype)
    pos = torch.arange(Tmax, device=q.device)[None, :]
    keep = pos < lens[:, None]
    if window:
        keep &= pos >= (lens[:, None] - int(window))
    n_rep = Hq // Hk
    kf = k_cache.float().repeat_interleave(n_rep, dim=2)   # [B, T, Hq, hd]
    vf = v_cache.float().repeat_interleave(n_rep, dim=2)
    s = torch.einsum("bhd,bthd->bht", q.float(), kf) * scale
    s = s.masked_fill(~keep[:, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("bht,bthd->bhd", p, vf).to(q.dtype)


def filter_logits(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None,
                  top_p: float | None = None) -> torch.Tensor:
    """Temperature, top-k (ties kept) and shifted top-p masking; returns fp32 logits with ``-inf`` holes."""
    z = logits.float() / max(float(temperature), 1e-6)
    if top_k is not None and 0 < int(top_k) < z.shape[-1]:
        kth = torch.topk(z, int(top_k)).values[..., -1:]
        z = z.masked_fill(z < kth, float("-inf"))
    if top_p is not None and 0 < float(top_p) < 1:
        sl, si = torch.sort(z, descending=True)
        sp = torch.softmax(sl, -1)
        drop = sp.cumsum(-1) - sp > float(top_p)
        sl = sl.masked_fill(drop, float("-inf"))
        z = torch.full_like(z, float("-inf")).scatter(-1, si, sl)
    return z


def sample_ref(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None, top_p: float | None = None,
               greedy: bool = False, generator: torch.Generator | None = None) -> torch.Tensor:
    if greedy or temperature <= 0:
        return logits.argmax(-1)
    z = filter_logits(logits, temperature, top_k, top_p)
    return torch.multinomial(torch.softmax(z, -1), 1, generator=generator).squeeze(-1)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int | None = None, top_p: float | None = None,
           greedy: bool = False, seed: int = 0, offset: int = 0, generator: torch.Generator | None = None) -> torch.Tensor:
    """Next tokens ``[B]`` (int64) from ``logits [B, V]``; one kernel launch on CUDA."""
    if logits.dim() != 2:
        logits = logits.reshape(-1, logits.shape[-1])
    if _kernel_ok(logits) and logits.dtype in (torch.float32, torch.bfloat16) and logits.stride(1) == 1 and generator is None:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
        rc = _lib.lib().ob_sample(_lib.ptr(logits), int(logits.dtype == torch.bfloat16), logits.stride(0), logits.shape[0],
                                  logits.shape[1], float(temperature), int(top_k or 0), float(top_p or 0.0), int(greedy),
                                  int(seed) & 0xFFFFFFFFFFFFFFFF, int(offset) & 0xFFFFFFFFFFFFFFFF, _lib.ptr(out),
                                  _lib.stream())
        _lib.check(rc, "ob_sample")
        return out
    return sample_ref(logits, temperature, top_k, top_p, greedy, generator)
