"""Feed-forward blocks (optimus_dl/modules/model/blocks/mlp.py:17-160).

``SwiGLUMLP`` keeps the reference's parameter names (``w1`` gate, ``w2`` up, ``c_proj`` down) and runs
the gate/up projections plus the activation as one dual-B tcgen05 GEMM on CUDA bf16.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import activation as act_ops
from ...ops import linear as lin_ops


def swiglu_hidden_dim(n_embd: int, intermediate_size: int | None, multiple_of: int) -> int:
    if intermediate_size is not None:
        return intermediate_size
    hidden = int(2 * (4 * n_embd) / 3)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


class SwiGLUMLP(nn.Module):
    def __init__(self, n_embd: int, intermediate_size: int | None = None, multiple_of: int = 256, bias: bool = False,
                 use_liger: bool | None = None, dropout: float = 0.0):
        super().__init__()
        hidden = swiglu_hidden_dim(n_embd, intermediate_size, multiple_of)
        self.w1 = nn.Linear(n_embd, hidden, bias=bias)
        self.w2 = nn.Linear(n_embd, hidden, bias=bias)
        self.c_proj = nn.Linear(hidden, n_embd, bias=bias)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        self.tp = None  # parallel.tp.TPState once the block is tensor-parallel

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``mlp(x)``, or ``residual + mlp(x)`` when a residual is given."""
        if self.tp is not None:
            from ...parallel import tp as tp_ops

            return tp_ops.swiglu_mlp_forward(self, x, residual)
        if residual is not None:
            return residual + self.forward(x)
        if lin_ops.fp8_route([self.w1.weight, self.w2.weight, self.c_proj.weight]):
            # FP8 context: gate/up as one block-scaled GEMM, SwiGLU, then the down projection
            gu = lin_ops.multi_linear(x, [self.w1.weight, self.w2.weight], [self.w1.bias, self.w2.bias])
            g, u = gu.split(self.w1.weight.shape[0], dim=-1)
            y = lin_ops.linear(act_ops.swiglu(g.contiguous(), u.contiguous()), self.c_proj.weight, self.c_proj.bias)
            return self.dropout(y) if self.dropout is not None else y
        if self.w1.bias is None and self.c_proj.bias is None:
            y = act_ops.swiglu_mlp(x, self.w1.weight, self.w2.weight, self.c_proj.weight)
            return self.dropout(y) if self.dropout is not None else y
        if self.w1.bias is None:
            h = act_ops.swiglu_mlp_up(x, self.w1.weight, self.w2.weight)
        else:
            h = act_ops.swiglu(lin_ops.linear(x, self.w1.weight, self.w1.bias),
                               lin_ops.linear(x, self.w2.weight, self.w2.bias))
        y = lin_ops.linear(h, self.c_proj.weight, self.c_proj.bias)
        return self.dropout(y) if self.dropout is not None else y


class ReLU2MLP(nn.Module):
    """``c_proj(relu(c_fc(x))^2)``."""

    def __init__(self, n_embd: int, intermediate_size: int | None = None, bias: bool = False, dropout: float = 0.0):
        super().__init__()
        hidden = intermediate_size or 4 * n_embd
        self.c_fc = nn.Linear(n_embd, hidden, bias=bias)
        self.c_proj = nn.Linear(hidden, n_embd, bias=bias)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        self.tp = None

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if self.tp is not None:
            from ...parallel import tp as tp_ops

            return tp_ops.dense_mlp_forward(self, x, lambda t: torch.relu(t).square(), residual)
        if residual is not None:
            return residual + self.forward(x)
        h = torch.relu(lin_ops.linear(x, self.c_fc.weight, self.c_fc.bias)).square()
        y = lin_ops.linear(h, self.c_proj.weight, self.c_proj.bias)
        return self.dropout(y) if self.dropout is not None else y


class GELUMLP(nn.Module):
    """``c_proj(gelu_erf(c_fc(x)))`` (GPT-2 style)."""

    def __init__(self, n_embd: int, intermediate_size: int | None = None, bias: bool = True, dropout: float = 0.0):
        super().__init__()
        hidden = intermediate_size or 4 * n_embd
        self.c_fc = nn.Linear(n_embd, hidden, bias=bias)
        self.c_proj = nn.Linear(hidden, n_embd, bias=bias)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        self.tp = None

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if self.tp is not None:
            from ...parallel import tp as tp_ops

            return tp_ops.dense_mlp_forward(self, x, torch.nn.functional.gelu, residual)
        if residual is not None:
            return residual + self.forward(x)
        h = torch.nn.functional.gelu(lin_ops.linear(x, self.c_fc.weight, self.c_fc.bias))
        y = lin_ops.linear(h, self.c_proj.weight, self.c_proj.bias)
        return self.dropout(y) if self.dropout is not None else y


def build_mlp(mlp_type: str, n_embd: int, intermediate_size: int | None, multiple_of: int, bias: bool,
              dropout: float = 0.0) -> nn.Module:
    if mlp_type == "swiglu":
        return SwiGLUMLP(n_embd, intermediate_size, multiple_of, bias, dropout=dropout)
    if mlp_type == "relu2":
        return ReLU2MLP(n_embd, intermediate_size, bias, dropout)
    if mlp_type == "gelu":
        return GELUMLP(n_embd, intermediate_size, bias, dropout)
    raise ValueError(f"unknown mlp_type {mlp_type!r}")
