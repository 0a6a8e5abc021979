"""Chunked fused linear + cross-entropy.

``linear_cross_entropy(x, W, targets)`` computes ``mean CE(x W^T, targets)`` without ever
holding the ``[tokens, vocab]`` logits: rows are processed in chunks; each chunk's logits come
from the tcgen05 GEMM, two kernels (``csrc/ce.cu``) turn them into per-row statistics and then,
in place, into ``d loss / d logits``; two more GEMMs give ``dX`` and accumulate ``dW``. The
backward pass therefore only rescales the stored gradients. When no gradient is asked for
(evaluation, metrics, the log-probability pass of the GRPO recipe) not even a chunk is written:
the GEMM's epilogue reduces its accumulator tiles to the statistics (``gemm.ce_stats_gemm``).

With a tensor-parallel group the weight is a vocabulary shard ``[V/tp, d]``; ranks exchange
``(max, sum-exp, target logit, sum of logits, arg max)`` per row (5 floats) instead of logits.

Loss definition (ignore index, label smoothing, tanh / sigmoid soft-capping, mean over valid
targets) follows optimus_dl/modules/criterion/cross_entropy.py:191-267 of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib, gemm

SOFTCAP = {None: 0, "none": 0, "tanh": 1, "sigmoid": 2}


def apply_softcap(logits: torch.Tensor, softcap: float | None, softcap_type: str = "tanh") -> torch.Tensor:
    if softcap is None and softcap_type != "sigmoid":
        return logits
    if softcap_type == "sigmoid":
        return 23.0 * torch.sigmoid((logits + 5.0) / 7.5)
    return softcap * torch.tanh(logits / softcap)


@dataclass
class CEResult:
    loss: torch.Tensor          # mean over valid targets (scalar, fp32, differentiable)
    n_valid: torch.Tensor       # number of non-ignored targets (scalar, int64)
    n_correct: torch.Tensor     # arg-max hits among valid targets (scalar, int64)
    loss_sum: torch.Tensor      # sum of per-token losses (scalar, fp32, detached)


def cross_entropy_ref(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100,
                      label_smoothing: float = 0.0, softcap: float | None = None, softcap_type: str = "tanh") -> CEResult:
    """fp32 PyTorch reference on materialised logits ``[rows, V]``."""
    z = logits.float()
    if softcap is not None or softcap_type == "sigmoid":
        z = apply_softcap(z, softcap, softcap_type)
    valid = targets != ignore_index
    loss_sum = F.cross_entropy(z, targets, ignore_index=ignore_index, label_smoothing=label_smoothing, reduction="sum")
    n_valid = valid.sum()
    n_correct = ((z.argmax(-1) == targets) & valid).sum()
    return CEResult(loss_sum / n_valid.clamp(min=1), n_valid, n_correct, loss_sum.detach())


class _LinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, targets, ignore_index, smoothing, softcap, softcap_type, chunk_rows, tp_group,
                vocab_offset, total_vocab, grad_scale):
        l = _lib.lib()
        dev = x.device
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        tg = targets.reshape(-1).to(torch.int64).contiguous()
        T = x2.shape[0]
        V = weight.shape[0]
        total_vocab = total_vocab or V
        mode = SOFTCAP["sigmoid" if softcap_type == "sigmoid" else ("tanh" if softcap is not None else None)]
        cap_c = float(softcap) if softcap is not None else 1.0
        valid = tg != ignore_index
        n_valid = valid.sum()
        inv_n = (1.0 / n_valid.clamp(min=1).float()).reshape(1)
        need_dx = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        dx = torch.empty_like(x2) if need_dx else None
        mg = getattr(weight, "main_grad", None) if need_dw else None
        if mg is not None:
            # accumulate straight into the sharding engine's flat gradient buffer (unit upstream
            # gradient is assumed: the criterion passes the loss scale through ``grad_scale``)
            dw = mg
            first_acc = bool(getattr(weight, "_main_grad_filled", False))
            weight._main_grad_filled = True
        else:
            dw = torch.empty_like(weight) if need_dw else None
            first_acc = False
        ld = (V + 7) // 8 * 8
        chunk_rows = min(chunk_rows, T)
        logits_buf = None                 # allocated when a chunk has to be materialised
        stats = torch.empty((5, T), dtype=torch.float32, device=dev)
        best_idx = torch.empty(T, dtype=torch.int32, device=dev)
        lse_all = torch.empty(T, dtype=torch.float32, device=dev)
        first = True
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            rows = r1 - r0
            # Without gradients (evaluation, metrics) the statistics come out of the GEMM's epilogue and no logits
            # are written; with gradients the bf16 chunk is needed anyway (it becomes d loss / d logits in place).
            st = stats[:, r0:r1]
            fused = not (need_dx or need_dw) and gemm.ce_stats_gemm(
                x2[r0:r1], weight, tg[r0:r1], st, best_idx[r0:r1], int(vocab_offset), mode, cap_c)
            if not fused:
                if logits_buf is None:
                    logits_buf = torch.empty((chunk_rows, ld), dtype=torch.bfloat16, device=dev)
                out_view = logits_buf[:rows].as_strided((rows, V), (ld, 1))
                gemm.gemm(x2[r0:r1], weight, out=out_view)
                rc = l.ob_ce_stats(_lib.ptr(out_view), ld, _lib.ptr(tg[r0:r1]), _lib.ptr(st[0]), _lib.ptr(st[1]),
                                   _lib.ptr(st[2]), _lib.ptr(st[3]), _lib.ptr(st[4]), _lib.ptr(best_idx[r0:r1]), rows, V,
                                   int(vocab_offset), mode, cap_c, _lib.stream())
                _lib.check(rc, "ob_ce_stats")
            mx, se, sz, zt, bv = st[0], st[1], st[2], st[3], st[4]
            if tp_group is not None:
                import torch.distributed as dist

                ws = dist.get_world_size(tp_group)
                pack = torch.stack([mx, se, sz, zt, bv, best_idx[r0:r1].float()], 0).contiguous()
                allp = torch.empty((ws, *pack.shape), dtype=pack.dtype, device=dev)
                dist.all_gather_into_tensor(allp, pack, group=tp_group)
                gmx = allp[:, 0].max(0).values
                gse = (allp[:, 1] * torch.exp(allp[:, 0] - gmx)).sum(0)
                sz = allp[:, 2].sum(0)
                zt = allp[:, 3].sum(0)
                bi = allp[:, 4].argmax(0, keepdim=True)
                best_idx[r0:r1] = allp[:, 5].gather(0, bi).squeeze(0).to(torch.int32)
                mx, se = gmx, gse
                stats[2, r0:r1] = sz
                stats[3, r0:r1] = zt
            lse = mx + torch.log(se)
            lse_all[r0:r1] = lse
            if need_dx or need_dw:
                rc = l.ob_ce_grad(_lib.ptr(out_view), ld, _lib.ptr(tg[r0:r1]), _lib.ptr(lse), rows, V, int(vocab_offset),
                                  int(total_vocab), int(ignore_index), float(smoothing), _lib.ptr(inv_n), float(grad_scale), mode,
                                  cap_c, None, _lib.stream())
                _lib.check(rc, "ob_ce_grad")
                if need_dx:
                    gemm.gemm(out_view, weight, b_mn=True, out=dx[r0:r1])
                if need_dw:
                    gemm.gemm(out_view, x2[r0:r1], a_mn=True, b_mn=True, out=dw, accumulate=(not first) or first_acc)
            first = False
        zt_all, sz_all = stats[3], stats[2]
        per_tok = lse_all - (1.0 - smoothing) * zt_all - smoothing * sz_all / total_vocab
        per_tok = torch.where(valid, per_tok, torch.zeros_like(per_tok))
        loss_sum = per_tok.sum()
        loss = loss_sum * inv_n[0]
        n_correct = ((best_idx.to(torch.int64) == tg) & valid).sum()
        if need_dx and tp_group is not None:
            import torch.distributed as dist

            dist.all_reduce(dx, group=tp_group)
        ctx.save_for_backward(dx if need_dx else torch.empty(0), dw if (need_dw and mg is None) else torch.empty(0))
        ctx.x_shape = x.shape
        ctx.grad_scale = float(grad_scale)
        ctx.flags = (need_dx, need_dw and mg is None)
        ctx.mark_non_differentiable(n_valid, n_correct, loss_sum)
        return loss, n_valid, n_correct, loss_sum

    @staticmethod
    def backward(ctx, dloss, *_):
        dx, dw = ctx.saved_tensors
        need_dx, need_dw = ctx.flags
        # gradients were computed with ``grad_scale`` folded in; a unit upstream gradient is the
        # common case (loss.backward()), anything else rescales here
        # (``grad_scale`` is the upstream gradient the caller promised, e.g. 1 / accumulation steps)
        factor = dloss / ctx.grad_scale
        gx = (dx * factor.to(dx.dtype)).view(ctx.x_shape) if need_dx else None
        gw = dw * factor.to(dw.dtype) if need_dw else None
        return gx, gw, None, None, None, None, None, None, None, None, None, None


class _LinearTokenLoss(torch.autograd.Function):
    """Sum of an arbitrary per-token loss of ``log p(target)`` under the head ``x W^T``.

    ``loss_fn(nll_chunk, r0, r1) -> (loss_chunk, dloss_dnll_chunk)`` is evaluated per row chunk
    between the statistics kernel and the gradient kernel, so losses whose per-token weight depends
    on the log-probability itself (clipped policy ratios, KL penalties) need one pass over the
    ``[tokens, vocab]`` logits, which are never held beyond a chunk.
    """

    @staticmethod
    def forward(ctx, x, weight, targets, loss_fn, chunk_rows):
        l = _lib.lib()
        dev = x.device
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        tg = targets.reshape(-1).to(torch.int64).contiguous()
        T, V = x2.shape[0], weight.shape[0]
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx = torch.empty_like(x2) if need_dx else None
        mg = getattr(weight, "main_grad", None) if need_dw else None
        if mg is not None:
            dw, first_acc = mg, bool(getattr(weight, "_main_grad_filled", False))
            weight._main_grad_filled = True
        else:
            dw, first_acc = (torch.empty_like(weight) if need_dw else None), False
        ld = (V + 7) // 8 * 8
        chunk_rows = min(chunk_rows, T)
        logits_buf = None                 # allocated when a chunk has to be materialised (gradients)
        st = torch.empty((5, chunk_rows), dtype=torch.float32, device=dev)
        best = torch.empty(chunk_rows, dtype=torch.int32, device=dev)
        nll_all = torch.empty(T, dtype=torch.float32, device=dev)
        total = torch.zeros((), dtype=torch.float32, device=dev)
        first = True
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            rows = r1 - r0
            fused = not (need_dx or need_dw) and gemm.ce_stats_gemm(x2[r0:r1], weight, tg[r0:r1], st[:, :rows],
                                                                     best[:rows], 0, 0, 1.0)
            if not fused:
                if logits_buf is None:
                    logits_buf = torch.empty((chunk_rows, ld), dtype=torch.bfloat16, device=dev)
                out_view = logits_buf[:rows].as_strided((rows, V), (ld, 1))
                gemm.gemm(x2[r0:r1], weight, out=out_view)
                rc = l.ob_ce_stats(_lib.ptr(out_view), ld, _lib.ptr(tg[r0:r1]), _lib.ptr(st[0]), _lib.ptr(st[1]),
                                   _lib.ptr(st[2]), _lib.ptr(st[3]), _lib.ptr(st[4]), _lib.ptr(best), rows, V, 0, 0, 1.0,
                                   _lib.stream())
                _lib.check(rc, "ob_ce_stats")
            lse = st[0, :rows] + torch.log(st[1, :rows])
            nll = lse - st[3, :rows]
            nll_all[r0:r1] = nll
            loss_chunk, dl_dnll = loss_fn(nll, r0, r1)
            total += loss_chunk.sum()
            if need_dx or need_dw:
                w_rows = dl_dnll.to(torch.float32).contiguous()
                rc = l.ob_ce_grad(_lib.ptr(out_view), ld, _lib.ptr(tg[r0:r1]), _lib.ptr(lse.contiguous()), rows, V, 0, V,
                                  -(1 << 62), 0.0, None, 1.0, 0, 1.0, _lib.ptr(w_rows), _lib.stream())
                _lib.check(rc, "ob_ce_grad")
                if need_dx:
                    gemm.gemm(out_view, weight, b_mn=True, out=dx[r0:r1])
                if need_dw:
                    gemm.gemm(out_view, x2[r0:r1], a_mn=True, b_mn=True, out=dw, accumulate=(not first) or first_acc)
            first = False
        ctx.save_for_backward(dx if need_dx else torch.empty(0), dw if (need_dw and mg is None) else torch.empty(0))
        ctx.x_shape = x.shape
        ctx.flags = (need_dx, need_dw and mg is None)
        ctx.mark_non_differentiable(nll_all)
        return total, nll_all

    @staticmethod
    def backward(ctx, dloss, _dnll):
        dx, dw = ctx.saved_tensors
        need_dx, need_dw = ctx.flags
        gx = (dx * dloss.to(dx.dtype)).view(ctx.x_shape) if need_dx else None
        gw = dw * dloss.to(dw.dtype) if need_dw else None
        return gx, gw, None, None, None


def linear_token_loss(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, loss_fn, chunk_rows: int = 4096):
    """``(sum_i loss_i, nll)`` where ``nll_i = -log softmax(x_i W^T)[target_i]`` and
    ``loss_fn(nll_chunk, r0, r1) -> (loss_chunk, dloss/dnll chunk)`` defines the per-token loss.

    The returned sum is differentiable with respect to ``x`` and ``weight`` (the gradient uses the
    derivative ``loss_fn`` reports, treated as exact); ``nll`` is detached. Every target must be a
    valid class: mask tokens through ``loss_fn`` (zero loss and zero derivative), not the target.
    """
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _LinearTokenLoss.apply(x, weight, targets, loss_fn, chunk_rows)
    logits = F.linear(x.reshape(-1, x.shape[-1]), weight).float()
    nll = F.cross_entropy(logits, targets.reshape(-1), reduction="none")
    loss_vals, dl = loss_fn(nll.detach(), 0, nll.numel())
    # same contract as the kernel path: the value comes from loss_fn, the gradient from its reported derivative
    total = loss_vals.sum().detach() + ((nll - nll.detach()) * dl.detach()).sum()
    return total, nll.detach()


class _SumGradOverGroup(torch.autograd.Function):
    """Identity forward; the gradient is summed over the group (replicated input of a sharded op)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, dy):
        import torch.distributed as dist

        dy = dy.contiguous().clone()
        dist.all_reduce(dy, group=ctx.group)
        return dy, None


class _GatherVocab(torch.autograd.Function):
    """All-gather of vocabulary shards along the last dimension; the gradient is sliced."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist

        ctx.group, ctx.cols = group, x.shape[-1]
        parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, dy):
        import torch.distributed as dist

        r = dist.get_rank(ctx.group)
        return dy[..., r * ctx.cols:(r + 1) * ctx.cols].contiguous(), None


def linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, *, ignore_index: int = -100,
                         label_smoothing: float = 0.0, softcap: float | None = None, softcap_type: str = "tanh",
                         chunk_rows: int = 4096, tp_group=None, vocab_offset: int = 0,
                         total_vocab: int | None = None, grad_scale: float = 1.0) -> CEResult:
    """Mean cross-entropy of ``x @ weight^T`` against ``targets`` (see module docstring)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        loss, n_valid, n_correct, loss_sum = _LinearCE.apply(x, weight, targets, ignore_index, label_smoothing, softcap,
                                                             softcap_type, chunk_rows, tp_group, vocab_offset, total_vocab,
                                                             grad_scale)
        return CEResult(loss, n_valid, n_correct, loss_sum)
    if tp_group is not None:
        # eager fallback (CPU / fp32): local logits, gathered over the vocabulary with autograd-aware collectives
        logits = _GatherVocab.apply(F.linear(_SumGradOverGroup.apply(x.reshape(-1, x.shape[-1]), tp_group), weight),
                                    tp_group)
        return cross_entropy_ref(logits, targets.reshape(-1), ignore_index, label_smoothing, softcap, softcap_type)
    logits = F.linear(x.reshape(-1, x.shape[-1]), weight)
    return cross_entropy_ref(logits, targets.reshape(-1), ignore_index, label_smoothing, softcap, softcap_type)
