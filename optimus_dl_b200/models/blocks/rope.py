"""Rotary-embedding helpers under the reference's module path (optimus_dl/modules/model/blocks/rope.py): the table
builder and the rotation live in ``ops.rope``; ``_reshape_for_broadcast`` is the shape helper for code that applies a
frequency table by hand."""

import torch

from ...ops.rope import apply_rotary_emb, precompute_freqs_cis  # noqa: F401


def _reshape_for_broadcast(freqs_cis: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """View ``freqs_cis`` so that it broadcasts against ``x``, whose layout is ``(B, T, heads, ...)``.

    A table without a batch dimension (``(T, ...)``, matching ``x`` on the sequence axis and on the trailing axes after
    the head axis) becomes ``(1, T, 1, ...)``; a per-sample table (``(B, T, ...)``, one dimension fewer than ``x``)
    becomes ``(B, T, 1, ...)``.
    """
    assert x.ndim >= 2, "x needs at least a batch / sequence layout"
    if freqs_cis.ndim == x.ndim - 1 and freqs_cis.shape[:2] == x.shape[:2]:
        assert freqs_cis.shape[2:] == x.shape[3:], (freqs_cis.shape, x.shape)
        return freqs_cis.unsqueeze(2)
    tail = x.shape[3:] if x.ndim > 3 else x.shape[-1:]
    assert freqs_cis.shape[0] == x.shape[1] and tuple(freqs_cis.shape[1:]) == tuple(tail), (freqs_cis.shape, x.shape)
    shape = [1, x.shape[1]] + [1] * max(0, x.ndim - 2 - len(tail)) + list(tail)
    return freqs_cis.view(*shape)
