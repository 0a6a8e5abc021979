"""``adamw`` (optimus_dl/modules/optim/adamw.py:13-57).

Parameters owned by the sharding engine get :class:`~optimus_dl_b200.parallel.fsdp.ShardedAdamW`
(fp32 master / moment shards updated inside the reduce-scatter kernel); CUDA parameters outside
the engine get :class:`FusedAdamW`, which runs this package's flat AdamW kernel per parameter with
fp32 state; CPU parameters fall back to ``torch.optim.AdamW``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..core.registry import RegistryConfigStrict
from ..ops import optim as optim_ops
from . import register_optimizer


@dataclass
class AdamWConfig(RegistryConfigStrict):
    lr: float = 1e-3
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 1e-2
    amsgrad: bool = False
    maximize: bool = False
    foreach: bool | None = None
    capturable: bool = False
    differentiable: bool = False
    fused: bool = True


def refuse_sharded(param_groups: list, who: str) -> None:
    """Optimizers that need the whole gradient of a parameter cannot run on parameters of the sharding engine:
    their gradients are reduced straight into per-rank fp32 shards and ``p.grad`` stays empty."""
    for group in param_groups:
        for p in group["params"]:
            if getattr(p, "_shard_group", None) is not None:
                raise ValueError(f"{who} needs full gradients and cannot be combined with the fully_shard transform "
                                 "(use ddp or a single GPU, or adamw with fully_shard)")


def strip_names(params: Any) -> Any:
    """Accept ``(name, param)`` tuples anywhere a parameter is expected."""
    def plain(p):
        return p[1] if isinstance(p, tuple) else p

    if isinstance(params, dict):
        return [dict(params, params=[plain(p) for p in params["params"]])]
    out = []
    for g in params:
        if isinstance(g, dict):
            out.append(dict(g, params=[plain(p) for p in g["params"]]))
        else:
            out.append(plain(g))
    return out


class FusedAdamW(torch.optim.Optimizer):
    """AdamW with fp32 master weights and moments, one kernel launch per parameter."""

    def __init__(self, params: Any, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2):
        super().__init__(strip_names(params), dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["master"] = p.detach().float().clone().view(-1)
                    st["exp_avg"] = torch.zeros_like(st["master"])
                    st["exp_avg_sq"] = torch.zeros_like(st["master"])
                st["step"] += 1
                g = p.grad.contiguous().view(-1)
                if p.dtype == torch.bfloat16 and p.is_contiguous():
                    optim_ops.adamw_step_(st["master"], st["exp_avg"], st["exp_avg_sq"], g, p.view(-1), lr=group["lr"],
                                          beta1=b1, beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"],
                                          step=st["step"])
                else:
                    optim_ops.adamw_step_(st["master"], st["exp_avg"], st["exp_avg_sq"], g, None, lr=group["lr"],
                                          beta1=b1, beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"],
                                          step=st["step"])
                    p.copy_(st["master"].view_as(p))
        return loss


@register_optimizer("adamw", AdamWConfig)
def make_adamw(cfg, params, **_):
    groups = strip_names(params)
    flat = [p for g in groups for p in (g["params"] if isinstance(g, dict) else [g])]
    engines = {getattr(p, "_shard_group", None) is not None for p in flat}
    if engines == {True}:
        from ..parallel.fsdp import ShardedAdamW

        engine = flat[0]._shard_group.engine
        return ShardedAdamW(groups, engine, lr=cfg.lr, betas=tuple(cfg.betas), eps=cfg.eps, weight_decay=cfg.weight_decay)
    if flat and all(p.is_cuda for p in flat):
        return FusedAdamW(groups, lr=cfg.lr, betas=tuple(cfg.betas), eps=cfg.eps, weight_decay=cfg.weight_decay)
    # parameters that are not all on the GPU: the library optimizer with the config's own flags
    # (optimus_dl/modules/optim/adamw.py:42-57)
    return torch.optim.AdamW(groups, lr=cfg.lr, betas=tuple(cfg.betas), eps=cfg.eps, weight_decay=cfg.weight_decay,
                             amsgrad=cfg.amsgrad, maximize=cfg.maximize, foreach=cfg.foreach,
                             capturable=cfg.capturable, differentiable=cfg.differentiable, fused=cfg.fused)
