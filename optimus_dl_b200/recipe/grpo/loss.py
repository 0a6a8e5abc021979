"""GRPO objective on per-token log-probabilities.

For a generated token with policy log-probability ``l``, sampling-time log-probability ``l_old``,
frozen-reference log-probability ``l_ref`` and group-normalised advantage ``A``:

    ratio   = exp(l - l_old)
    policy  = -min(ratio * A, clip(ratio, 1 - eps, 1 + eps) * A)
    kl      = exp(l_ref - l) - (l_ref - l) - 1            (non-negative "k3" estimator)
    loss    = (policy + beta * kl) * mask / n_tokens

``token_loss`` returns the loss values together with their exact derivative with respect to the
negative log-likelihood ``nll = -l``, which is what ``ops.cross_entropy.linear_token_loss`` feeds
to the fused head kernels.
"""

from __future__ import annotations

import torch


def group_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-6) -> torch.Tensor:
    """``(r - mean_group) / (std_group + eps)`` for rewards laid out as consecutive groups."""
    r = rewards.view(-1, group_size).float()
    adv = (r - r.mean(-1, keepdim=True)) / (r.std(-1, unbiased=False, keepdim=True) + eps)
    return adv.reshape(-1)


def token_loss(nll: torch.Tensor, old_logp: torch.Tensor, ref_logp: torch.Tensor | None, adv: torch.Tensor,
               mask: torch.Tensor, clip_eps: float, kl_coef: float, inv_tokens: float):
    """Returns ``(loss, dloss_dnll, stats)`` for flat per-token tensors of equal length."""
    logp = -nll.float()
    ratio = torch.exp(logp - old_logp)
    unclipped = ratio * adv
    clipped = ratio.clamp(1.0 - clip_eps, 1.0 + clip_eps) * adv
    use_unclipped = unclipped <= clipped
    policy = -torch.where(use_unclipped, unclipped, clipped)
    # d policy / d logp: -A * ratio where the unclipped branch is active or the clip is not binding, else 0
    inside = (ratio >= 1.0 - clip_eps) & (ratio <= 1.0 + clip_eps)
    dpolicy = torch.where(use_unclipped | inside, -adv * ratio, torch.zeros_like(ratio))
    m = mask.float()
    if ref_logp is not None and kl_coef:
        d = ref_logp - logp
        kl = torch.exp(d) - d - 1.0
        dkl = 1.0 - torch.exp(d)          # d kl / d logp
    else:
        kl = torch.zeros_like(logp)
        dkl = torch.zeros_like(logp)
    loss = (policy + kl_coef * kl) * m * inv_tokens
    dloss_dlogp = (dpolicy + kl_coef * dkl) * m * inv_tokens
    stats = {"kl_sum": (kl * m).sum(), "clipped_sum": ((~inside).float() * m).sum(), "ratio_sum": (ratio * m).sum()}
    return loss, -dloss_dlogp, stats
