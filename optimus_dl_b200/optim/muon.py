"""``muon``: momentum + Newton-Schulz orthogonalised updates for matrices, a support optimizer for
everything else (optimus_dl/modules/optim/muon.py:37-117).

The reference wraps ``torch.optim.Muon``; here the optimizer is implemented directly so that the
five Newton-Schulz iterations — three matrix products each, all of the ``A B^T`` / ``A B`` forms the
tcgen05 GEMM offers — run on this package's kernel for CUDA bf16 (``ops/gemm.py``) with the
``b A + c A A`` and ``a X + B X`` sums folded into the GEMM epilogue (scale + accumulate).
Update rule and defaults match ``torch.optim.Muon``: ``buf = mu * buf + (1 - mu) * g``; the update is
``lerp(g, buf, mu)`` with Nesterov, else ``buf``; ``p *= 1 - lr * wd``;
``p -= adjusted_lr * orthogonalise(update)``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch
from torch.optim.optimizer import Optimizer

from ..core.conf import II
from ..core.registry import RegistryConfigStrict
from ..ops import gemm
from . import build_optimizer, register_optimizer
from .adamw import refuse_sharded, strip_names
from .composite import CompositeOptimizer, get_subgroup

DEFAULT_NS_COEFFICIENTS = (3.4445, -4.7750, 2.0315)
DEFAULT_NS_STEPS = 5
EPS = 1e-7


@dataclass
class MuonConfig(RegistryConfigStrict):
    lr: float = 1e-3
    weight_decay: float = 0.1
    momentum: float = 0.95
    nesterov: bool = True
    ns_coefficients: tuple[float, float, float] = DEFAULT_NS_COEFFICIENTS
    eps: float = EPS
    ns_steps: int = DEFAULT_NS_STEPS
    adjust_lr_fn: str | None = None
    support_optimizer: Any = field(default_factory=lambda: {
        "_name": "adamw", "lr": II("..lr"), "weight_decay": II("..weight_decay"), "eps": II("..eps")})


def newton_schulz(g: torch.Tensor, steps: int = DEFAULT_NS_STEPS, coefficients=DEFAULT_NS_COEFFICIENTS,
                  eps: float = EPS) -> torch.Tensor:
    """Approximate ``U V^T`` of ``g = U S V^T`` with the quintic Newton-Schulz iteration, in bf16."""
    assert g.dim() == 2
    a, b, c = (float(v) for v in coefficients)
    x = g.to(torch.bfloat16)
    tall = x.shape[0] > x.shape[1]
    if tall:
        x = x.t()
    x = (x / (x.float().norm() + eps).to(x.dtype)).contiguous()
    fused = x.is_cuda and x.shape[0] % 8 == 0 and x.shape[1] % 8 == 0
    for _ in range(int(steps)):
        if fused:
            aa = gemm.gemm(x, x)                                           # A = X X^T (symmetric)
            bm = aa * b
            gemm.gemm(aa, aa, out=bm, alpha=c, accumulate=True)            # B = b A + c A A
            nx = x * a
            gemm.gemm(bm, x, b_mn=True, out=nx, accumulate=True)           # X = a X + B X
            x = nx
        else:
            aa = x @ x.t()
            bm = b * aa + c * (aa @ aa)
            x = a * x + bm @ x
    return x.t() if tall else x


def adjusted_lr(lr: float, shape: torch.Size, adjust_lr_fn: str | None) -> float:
    rows, cols = shape[0], shape[1]
    if adjust_lr_fn is None or adjust_lr_fn == "original":
        return lr * math.sqrt(max(1.0, rows / cols))
    if adjust_lr_fn == "match_rms_adamw":
        return lr * 0.2 * math.sqrt(max(rows, cols))
    raise ValueError(f"unknown adjust_lr_fn {adjust_lr_fn!r}")


class Muon(Optimizer):
    def __init__(self, params: Any, lr: float = 1e-3, weight_decay: float = 0.1, momentum: float = 0.95,
                 nesterov: bool = True, ns_coefficients=DEFAULT_NS_COEFFICIENTS, eps: float = EPS,
                 ns_steps: int = DEFAULT_NS_STEPS, adjust_lr_fn: str | None = None):
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov,
                        ns_coefficients=tuple(ns_coefficients), eps=eps, ns_steps=ns_steps, adjust_lr_fn=adjust_lr_fn)
        super().__init__(strip_names(params), defaults)
        refuse_sharded(self.param_groups, "Muon")
        for group in self.param_groups:
            for p in group["params"]:
                if p.dim() != 2:
                    raise ValueError(f"Muon only supports 2D parameters, got shape {tuple(p.shape)}")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            mu = group["momentum"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p.grad, memory_format=torch.preserve_format)
                buf = st["momentum_buffer"]
                buf.lerp_(p.grad, 1 - mu)
                upd = p.grad.lerp(buf, mu) if group["nesterov"] else buf
                ortho = newton_schulz(upd, group["ns_steps"], group["ns_coefficients"], group["eps"])
                p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(ortho.to(p.dtype), alpha=-adjusted_lr(group["lr"], p.shape, group["adjust_lr_fn"]))
        return loss


@register_optimizer("muon", MuonConfig)
def make_muon(cfg: Any, params: Any, **kwargs: Any):
    params = list(params)
    matrices = get_subgroup(params, lambda n, p: p.ndim == 2)
    others = get_subgroup(params, lambda n, p: p.ndim != 2)
    if not matrices:
        raise ValueError("Muon optimizer requires at least one 2D parameter (matrix).")
    muon = Muon(matrices, lr=float(cfg.lr), weight_decay=float(cfg.weight_decay), momentum=float(cfg.momentum),
                nesterov=bool(cfg.nesterov), ns_coefficients=tuple(cfg.ns_coefficients), eps=float(cfg.eps),
                ns_steps=int(cfg.ns_steps), adjust_lr_fn=getattr(cfg, "adjust_lr_fn", None))
    if not others:
        return muon
    support = build_optimizer(cfg.support_optimizer, params=others, **kwargs)
    return CompositeOptimizer({"muon": muon, "support": support})
