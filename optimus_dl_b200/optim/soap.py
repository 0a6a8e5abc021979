"""``soap``: Adam run in the eigenbasis of Shampoo's Kronecker factors (Vyas et al., arXiv:2409.11321;
configuration as optimus_dl/modules/optim/soap.py:20-100).

Per parameter (optionally reshaped by ``merge_dims``), each dimension ``i`` no larger than
``max_precond_dim`` keeps a factor ``GG_i = EMA(G_(i) G_(i)^T)`` and an orthonormal basis ``Q_i``.
Every step: the gradient is rotated into the basis, Adam's second moment lives there, the first
moment lives in parameter space and is rotated on use, and the Adam direction is rotated back.
Every ``precondition_frequency`` steps ``Q_i`` is refreshed with one power-iteration + QR step
(columns re-sorted by estimated eigenvalue, the second moment permuted alongside); the very first
step only initialises the factors with an eigendecomposition and does not move the parameter.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
from torch.optim.optimizer import Optimizer

from ..core.registry import RegistryConfigStrict
from . import register_optimizer
from .adamw import refuse_sharded, strip_names


@dataclass
class SoapConfig(RegistryConfigStrict):
    lr: float = 3e-3
    betas: tuple[float, float] = (0.95, 0.95)
    shampoo_beta: float = -1
    eps: float = 1e-8
    weight_decay: float = 0.01
    precondition_frequency: int = 10
    max_precond_dim: int = 10000
    merge_dims: bool = False
    precondition_1d: bool = False
    normalize_grads: bool = False
    data_format: str = "channels_first"
    correct_bias: bool = True


def merged_shape(shape: tuple[int, ...], limit: int) -> list[int]:
    """Greedily fold neighbouring dimensions while their product stays within ``limit``."""
    out: list[int] = []
    run = 1
    for s in shape:
        if run * s > limit:
            if run > 1:
                out.append(run)
                run = s
            else:
                out.append(s)
                run = 1
        else:
            run *= s
    if run > 1 or not out:
        out.append(run)
    return out


def _mode_product(t: torch.Tensor, q: torch.Tensor | None, transpose: bool) -> torch.Tensor:
    """Contract the leading axis of ``t`` with ``q`` (or just rotate the axes) and move it last: applying this
    once per axis returns to the original axis order. The columns of ``q`` are eigenvectors, so coordinates in the
    eigenbasis are ``q^T t`` (``transpose=False``: into the basis) and ``q t`` leads back (``transpose=True``)."""
    if q is None:
        return t.movedim(0, -1)
    return torch.tensordot(t, q, dims=([0], [1] if transpose else [0]))


class SOAP(Optimizer):
    def __init__(self, params: Any, lr: float = 3e-3, betas=(0.95, 0.95), shampoo_beta: float = -1, eps: float = 1e-8,
                 weight_decay: float = 0.01, precondition_frequency: int = 10, max_precond_dim: int = 10000,
                 merge_dims: bool = False, precondition_1d: bool = False, normalize_grads: bool = False,
                 data_format: str = "channels_first", correct_bias: bool = True):
        assert data_format in ("channels_first", "channels_last")
        defaults = dict(lr=lr, betas=tuple(betas), shampoo_beta=shampoo_beta, eps=eps, weight_decay=weight_decay,
                        precondition_frequency=precondition_frequency, max_precond_dim=max_precond_dim,
                        merge_dims=merge_dims, precondition_1d=precondition_1d, normalize_grads=normalize_grads,
                        correct_bias=correct_bias)
        super().__init__(strip_names(params), defaults)
        refuse_sharded(self.param_groups, "SOAP")
        self._data_format = data_format

    # ------------------------------------------------------------------ geometry
    def _view(self, g: torch.Tensor, group: dict) -> torch.Tensor:
        if not group["merge_dims"]:
            return g
        if self._data_format == "channels_last" and g.dim() == 4:
            g = g.permute(0, 3, 1, 2)
        return g.reshape(merged_shape(tuple(g.shape), int(group["max_precond_dim"])))

    def _unview(self, t: torch.Tensor, like: torch.Tensor, group: dict) -> torch.Tensor:
        if not group["merge_dims"]:
            return t
        if self._data_format == "channels_last" and like.dim() == 4:
            n, h, w, c = like.shape
            return t.reshape(n, c, h, w).permute(0, 2, 3, 1)
        return t.reshape(like.shape)

    @staticmethod
    def _rotate(t: torch.Tensor, bases: list, back: bool) -> torch.Tensor:
        for q in bases:
            t = _mode_product(t, q, transpose=back)
        return t

    def _init_factors(self, st: dict, gv: torch.Tensor, group: dict) -> None:
        limit = int(group["max_precond_dim"])
        if gv.dim() == 1 and not group["precondition_1d"]:
            st["GG"] = [None]
        else:
            st["GG"] = [torch.zeros(s, s, device=gv.device, dtype=torch.float32) if s <= limit else None for s in gv.shape]
        st["Q"] = None

    @staticmethod
    def _accumulate_factors(st: dict, gv: torch.Tensor, beta: float) -> None:
        gf = gv.float()
        for i, gg in enumerate(st["GG"]):
            if gg is None:
                continue
            rest = [d for d in range(gf.dim()) if d != i]
            outer = torch.tensordot(gf, gf, dims=(rest, rest)) if rest else torch.outer(gf, gf)
            gg.lerp_(outer, 1 - beta)

    @staticmethod
    def _eigenbases(factors: list) -> list:
        out = []
        for gg in factors:
            if gg is None:
                out.append(None)
                continue
            m = gg + 1e-30 * torch.eye(gg.shape[0], device=gg.device, dtype=gg.dtype)
            try:
                _, q = torch.linalg.eigh(m)
            except Exception:  # noqa: BLE001 - ill-conditioned in fp32
                _, q = torch.linalg.eigh(m.double())
                q = q.to(gg.dtype)
            out.append(q.flip(1).contiguous())   # eigenvalues descending
        return out

    def _refresh_bases(self, st: dict) -> None:
        """One step of orthogonal (power) iteration per factor, keeping the second moment aligned."""
        v = st["exp_avg_sq"]
        new_q = []
        for i, (gg, q) in enumerate(zip(st["GG"], st["Q"])):
            if gg is None:
                new_q.append(None)
                continue
            est = torch.einsum("ij,ij->j", q, gg @ q)     # diag(Q^T GG Q)
            order = torch.argsort(est, descending=True)
            v = v.index_select(i, order)
            qn, _ = torch.linalg.qr(gg @ q[:, order])
            new_q.append(qn.contiguous())
        st["Q"] = new_q
        st["exp_avg_sq"] = v

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            sb = group["shampoo_beta"] if group["shampoo_beta"] >= 0 else b2
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                st = self.state[p]
                gv = self._view(g, group)
                if "step" not in st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(g, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros(gv.shape, dtype=torch.float32, device=g.device)
                    self._init_factors(st, gv, group)
                if st["Q"] is None:
                    # first call: seed the factors and their bases, leave the parameter alone
                    self._accumulate_factors(st, gv, sb)
                    st["Q"] = self._eigenbases(st["GG"])
                    continue
                st["step"] += 1
                t = st["step"]
                g_rot = self._rotate(gv.float(), st["Q"], back=False)
                st["exp_avg"].lerp_(g.float(), 1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g_rot, g_rot, value=1 - b2)
                m_rot = self._rotate(self._view(st["exp_avg"], group), st["Q"], back=False)
                denom = st["exp_avg_sq"].sqrt().add_(group["eps"])
                step_size = group["lr"]
                if group["correct_bias"]:
                    step_size *= ((1 - b2 ** t) ** 0.5) / (1 - b1 ** t)
                direction = self._rotate(m_rot / denom, st["Q"], back=True)
                direction = self._unview(direction, g, group)
                if group["normalize_grads"]:
                    direction = direction / (1e-30 + direction.pow(2).mean().sqrt())
                p.add_(direction.to(p.dtype), alpha=-step_size)
                if group["weight_decay"] > 0:
                    p.add_(p, alpha=-group["lr"] * group["weight_decay"])
                self._accumulate_factors(st, gv, sb)
                if t % int(group["precondition_frequency"]) == 0:
                    self._refresh_bases(st)
        return loss


@register_optimizer("soap", SoapConfig)
def make_soap(cfg: Any, params: Any, **_: Any) -> SOAP:
    return SOAP(params, lr=float(cfg.lr), betas=tuple(cfg.betas), shampoo_beta=float(cfg.shampoo_beta), eps=float(cfg.eps),
                weight_decay=float(cfg.weight_decay), precondition_frequency=int(cfg.precondition_frequency),
                max_precond_dim=int(cfg.max_precond_dim), merge_dims=bool(cfg.merge_dims),
                precondition_1d=bool(cfg.precondition_1d), normalize_grads=bool(cfg.normalize_grads),
                data_format=str(cfg.data_format), correct_bias=bool(cfg.correct_bias))
