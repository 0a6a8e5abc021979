"""LayerNorm / RMSNorm modules (optimus_dl/modules/model/blocks/layer_norms.py:21-120).

CUDA bf16 inputs run ``csrc/norm.cu``; other inputs run the fp32 PyTorch formula. The
``use_liger`` flag of the reference is accepted and ignored (there is one kernel path here).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import norm as norm_ops


class LayerNorm(nn.Module):
    """LayerNorm with optional bias; eps fixed at 1e-5 like the reference."""

    def __init__(self, ndim: int, bias: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ndim))
        self.bias = nn.Parameter(torch.zeros(ndim)) if bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return norm_ops.layer_norm(x, self.weight, self.bias, 1e-5)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, use_liger: bool | None = None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        """``rmsnorm(x) * w``; with ``residual`` returns ``(rmsnorm(x + residual) * w, x + residual)``."""
        emit = False
        if getattr(self, "_fp8_out", False) and x.is_cuda:
            # marked by the transformer_engine transform: the consumers are FP8 linear layers with 1x128 scales
            from ...amp.fp8 import fp8_enabled
            from ...ops import fp8 as fp8_ops

            emit = fp8_enabled() and fp8_ops.scaling_mode() == "block"
        return norm_ops.rms_norm(x, self.weight, self.eps, residual, emit_fp8=emit)

    def _norm(self, x: torch.Tensor) -> torch.Tensor:
        """``x / rms(x)`` without the weight (the helper of optimus_dl/modules/model/blocks/layer_norms.py:86-96);
        ``forward`` does not go through it."""
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)

    def extra_repr(self) -> str:
        return f"{self.weight.numel()}, eps={self.eps}"
