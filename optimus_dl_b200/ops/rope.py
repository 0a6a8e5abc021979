"""Rotary position embeddings: frequency tables, the PyTorch reference and raw kernel calls.

Layout is *interleaved pairs*: ``(x0, x1), (x2, x3), ...`` are rotated together, and the
table has shape ``(max_pos, head_dim // 2, 2)`` holding ``(cos, sin)`` in fp32 — the same
contract as optimus_dl/modules/model/blocks/rope.py:13-118,181-253 in the reference
(including its ``yarn`` and ``llama3`` frequency scaling rules).
"""

from __future__ import annotations

import math

import torch

from . import _lib


def _yarn_inv_freq(dim: int, theta: float, base_inv: torch.Tensor, cfg: dict) -> tuple[torch.Tensor, float]:
    factor = cfg.get("factor", 1.0)
    orig = cfg.get("original_max_position_embeddings", 8192)
    att = cfg.get("attention_factor", 1.0)
    beta_fast = cfg.get("beta_fast", 32.0)
    beta_slow = cfg.get("beta_slow", 1.0)

    def corr_dim(rot: float) -> float:
        return dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    keep = 1.0 - ramp  # 1 => keep the original frequency (extrapolate), 0 => interpolate
    inv = (base_inv / factor) * (1.0 - keep) + base_inv * keep
    return inv, att


def _llama3_inv_freq(base_inv: torch.Tensor, cfg: dict) -> torch.Tensor:
    factor = cfg.get("factor", 8.0)
    lo_f = cfg.get("low_freq_factor", 1.0)
    hi_f = cfg.get("high_freq_factor", 4.0)
    old_len = cfg.get("original_max_position_embeddings", 8192)
    wavelen = 2 * math.pi / base_inv
    scale = torch.ones_like(base_inv)
    scale[wavelen > old_len / lo_f] = factor
    mid = (wavelen <= old_len / lo_f) & (wavelen >= old_len / hi_f)
    smooth = (old_len / wavelen[mid] - lo_f) / (hi_f - lo_f)
    scale[mid] = 1.0 + smooth * (factor - 1.0)
    return base_inv / scale


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0, scaling_config: dict | None = None) -> torch.Tensor:
    """``(end, dim // 2, 2)`` table of ``(cos, sin)``; optional ``yarn`` / ``llama3`` scaling."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    att = 1.0
    if scaling_config is not None:
        kind = scaling_config.get("rope_type")
        if kind == "yarn":
            inv, att = _yarn_inv_freq(dim, theta, inv, scaling_config)
        elif kind == "llama3":
            inv = _llama3_inv_freq(inv, scaling_config)
    ang = torch.outer(torch.arange(end), inv).float()
    return torch.stack((torch.cos(ang) * att, torch.sin(ang) * att), dim=-1)


def rotate_ref(x: torch.Tensor, freqs: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate ``x (..., T, H, hd)`` by ``freqs`` ``(T, hd/2, 2)`` or ``(B, T, hd/2, 2)`` in fp32."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    f = freqs.to(x.device)
    f = f[None, :, None] if f.dim() == 3 else f[:, :, None]  # -> (1|B, T, 1, hd/2, 2)
    c, s = f[..., 0], f[..., 1]
    if inverse:
        s = -s
    o0 = xf[..., 0] * c - xf[..., 1] * s
    o1 = xf[..., 0] * s + xf[..., 1] * c
    return torch.stack((o0, o1), dim=-1).flatten(-2).to(x.dtype)


def apply_rotary_emb(q: torch.Tensor, k: torch.Tensor, freqs_cis: torch.Tensor, position_ids: torch.Tensor | None = None):
    """PyTorch reference: rotate ``q`` and ``k`` of shape ``(B, T, H, hd)``."""
    T = q.shape[1]
    f = freqs_cis.to(q.device)
    f = f[position_ids] if position_ids is not None else f[:T]
    return rotate_ref(q, f), rotate_ref(k, f)


def rope_kernel_fwd(src: torch.Tensor, dst: torch.Tensor, src_stride: int, dst_stride: int, freqs: torch.Tensor,
                    pos_ids: torch.Tensor | None, qw, kw, rstd, T: int, Hq: int, Hk: int, hd: int, seq_len: int,
                    eps: float) -> None:
    """Raw launch: rotate ``Hq + Hk`` heads per token starting at ``src`` (token stride in elements)."""
    rc = _lib.lib().ob_qknorm_rope_fwd(_lib.ptr(src), _lib.ptr(dst), src_stride, dst_stride, _lib.ptr(freqs),
                                       _lib.ptr(pos_ids), _lib.ptr(qw), _lib.ptr(kw), _lib.ptr(rstd), T, Hq, Hk, hd,
                                       seq_len, float(eps), _lib.stream())
    _lib.check(rc, "ob_qknorm_rope_fwd")


def rope_kernel_bwd(dout: torch.Tensor, din: torch.Tensor, dout_stride: int, din_stride: int, x_in, x_stride: int,
                    freqs: torch.Tensor, pos_ids, qw, kw, rstd, dw_partial, T: int, Hq: int, Hk: int, hd: int,
                    seq_len: int) -> None:
    rc = _lib.lib().ob_qknorm_rope_bwd(_lib.ptr(dout), _lib.ptr(din), dout_stride, din_stride, _lib.ptr(x_in), x_stride,
                                       _lib.ptr(freqs), _lib.ptr(pos_ids), _lib.ptr(qw), _lib.ptr(kw), _lib.ptr(rstd),
                                       _lib.ptr(dw_partial), T, Hq, Hk, hd, seq_len, _lib.stream())
    _lib.check(rc, "ob_qknorm_rope_bwd")


def rope_grid(items: int) -> int:
    return int(_lib.lib().ob_rope_grid(items))
