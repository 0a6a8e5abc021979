"""Re-exports of the rotary-embedding helpers under the reference's module path
(optimus_dl/modules/model/blocks/rope.py)."""

from ...ops.rope import apply_rotary_emb, precompute_freqs_cis  # noqa: F401
