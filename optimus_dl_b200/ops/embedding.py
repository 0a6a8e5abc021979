"""Embedding lookup and its deterministic gradient (``csrc/elementwise.cu``).

The gradient sorts the token ids and lets one CTA add all rows of an id in a fixed order,
so repeated ids give bitwise-reproducible results without atomics.
Replaces ATen's embedding used by optimus_dl/modules/model/llama2.py:371.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, pad_id):
        ids64 = ids.reshape(-1).to(torch.int64).contiguous()
        T = ids64.numel()
        V, D = table.shape
        out = torch.empty((T, D), dtype=table.dtype, device=table.device)
        _lib.check(_lib.lib().ob_embedding_fwd(_lib.ptr(ids64), _lib.ptr(table), _lib.ptr(out), T, D, V, _lib.stream()),
                   "ob_embedding_fwd")
        ctx.save_for_backward(ids64)
        ctx.table_shape = (V, D)
        ctx.pad_id = -1 if pad_id is None else int(pad_id)
        ctx.table = table  # for main_grad lookup
        return out.view(*ids.shape, D)

    @staticmethod
    def backward(ctx, dout):
        (ids64,) = ctx.saved_tensors
        V, D = ctx.table_shape
        sorted_ids, perm = torch.sort(ids64, stable=True)
        d2 = dout.reshape(-1, D).contiguous()
        mg = getattr(ctx.table, "main_grad", None)
        if mg is not None:
            # scatter straight into the sharding engine's flat gradient buffer
            if not getattr(ctx.table, "_main_grad_filled", False):
                mg.zero_()
                ctx.table._main_grad_filled = True
            dtable, acc, ret = mg, 1, None
        else:
            dtable = torch.zeros((V, D), dtype=dout.dtype, device=dout.device)
            acc, ret = 0, dtable
        _lib.check(_lib.lib().ob_embedding_bwd(_lib.ptr(sorted_ids), _lib.ptr(perm), _lib.ptr(d2), _lib.ptr(dtable),
                                               ids64.numel(), D, V, ctx.pad_id, acc, _lib.stream()), "ob_embedding_bwd")
        return None, ret, None


def embedding(ids: torch.Tensor, table: torch.Tensor, padding_idx: int | None = None) -> torch.Tensor:
    if table.is_cuda and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0 and table.is_contiguous():
        return _Embedding.apply(ids, table, padding_idx)
    return F.embedding(ids, table, padding_idx)
