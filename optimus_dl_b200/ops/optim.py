"""Fused AdamW over flat fp32 shards and the deterministic sum of squares used for the global
gradient norm (``csrc/elementwise.cu``). Update rule = ``torch.optim.AdamW`` (decoupled weight
decay, bias correction), which the reference calls with ``fused=True``
(optimus_dl/modules/optim/adamw.py:45-57).
"""

from __future__ import annotations

import torch

from . import _lib

_scratch: dict[int, torch.Tensor] = {}


def _sumsq_scratch(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _scratch.get(idx)
    if buf is None:
        buf = torch.zeros(1026, dtype=torch.float32, device=device)
        _scratch[idx] = buf
    return buf


def sumsq_(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """``out[0] (+)= sum(x^2)``; ``out`` is a 1-element fp32 tensor on the same device."""
    x = x.contiguous().view(-1)
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32):
        rc = _lib.lib().ob_sumsq(_lib.ptr(x), x.numel(), int(x.dtype == torch.float32), _lib.ptr(_sumsq_scratch(x.device)),
                                 _lib.ptr(out), int(accumulate), _lib.stream())
        _lib.check(rc, "ob_sumsq")
    else:
        s = x.float().pow(2).sum()
        if accumulate:
            out.add_(s)
        else:
            out.fill_(s)
    return out


def adamw_step_(master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, grad: torch.Tensor,
                param_lp: torch.Tensor | None, *, lr: float, beta1: float, beta2: float, eps: float,
                weight_decay: float, step: int, grad_scale: float = 1.0, sumsq: torch.Tensor | None = None,
                max_norm: float = 0.0) -> None:
    """One AdamW step on flat tensors, in place.

    ``master``/``exp_avg``/``exp_avg_sq`` are fp32; ``grad`` is bf16 or fp32; ``param_lp`` (optional) is the
    bf16 copy refreshed from the new master value. With ``sumsq`` (device scalar holding the squared global
    gradient norm before ``grad_scale``) the gradient is clipped to ``max_norm`` inside the kernel.
    """
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    n = master.numel()
    if master.is_cuda and master.dtype == torch.float32 and grad.dtype in (torch.bfloat16, torch.float32):
        rc = _lib.lib().ob_adamw(_lib.ptr(master), _lib.ptr(exp_avg), _lib.ptr(exp_avg_sq), _lib.ptr(grad),
                                 int(grad.dtype == torch.float32), _lib.ptr(param_lp), n, lr, beta1, beta2, eps,
                                 weight_decay, bc1, bc2, grad_scale, _lib.ptr(sumsq), float(max_norm), _lib.stream())
        _lib.check(rc, "ob_adamw")
        return
    g = grad.float() * grad_scale
    if sumsq is not None:
        norm = sumsq.float().sqrt() * grad_scale
        g = g * torch.clamp(max_norm / (norm + 1e-6), max=1.0)
    master.mul_(1.0 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    denom = exp_avg_sq.sqrt() / (bc2 ** 0.5) + eps
    master.addcdiv_(exp_avg, denom, value=-lr / bc1)
    if param_lp is not None:
        param_lp.copy_(master)
