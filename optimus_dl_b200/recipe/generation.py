"""Autoregressive generation with a key/value cache.

The reference re-runs the full prefix for every new token, both in its ``generation`` metric source
(optimus_dl/modules/metrics/sources/generation.py:97-160) and in the serve recipe
(optimus_dl/recipe/serve/base.py). ``generate`` keeps that call contract (prompt ids in, new ids
out, per-sequence EOS stop with padding, greedy / temperature / top-k / top-p) but runs one prefill
and then single-token steps over per-layer caches: cached keys and values are read once per step
by ``ops.decode.decode_attention`` and the next token comes from the fused sampler.

On CUDA the decode step's launch sequence is identical from step to step (lengths and positions
live in device tensors), so it is captured once into a CUDA graph and replayed.
"""

from __future__ import annotations

import contextlib
import logging
from typing import Any, Iterator

import torch
import torch.nn as nn

from ..ops import decode as dec_ops

logger = logging.getLogger(__name__)


class LayerKV:
    """One attention layer's cache ``[B, Tmax, Hk, hd]`` plus the session state shared by all layers."""

    def __init__(self, session: "DecodeSession", k: torch.Tensor, v: torch.Tensor):
        self._s = session
        self.k, self.v = k, v
        self.workspace: dict = {}

    @property
    def seq_lens(self) -> torch.Tensor:
        return self._s.seq_lens

    @property
    def filled(self) -> bool:
        return self._s.filled

    @property
    def n_splits(self) -> int:
        return self._s.n_splits


def _attention_modules(model: nn.Module) -> list[nn.Module]:
    blocks = getattr(getattr(model, "transformer", None), "h", None)
    if blocks is None:
        return []
    mods = []
    for b in blocks:
        attn = getattr(b, "attn", None)
        if attn is None or not hasattr(attn, "_forward_cached"):
            return []
        mods.append(attn)
    return mods


def unwrap(model: nn.Module) -> nn.Module:
    m = model
    for _ in range(4):
        if hasattr(m, "transformer"):
            return m
        inner = getattr(m, "module", None)
        if inner is None:
            break
        m = inner
    return m


def supports_kv_cache(model: nn.Module) -> bool:
    m = unwrap(model)
    return bool(_attention_modules(m)) and getattr(m, "_tp", None) is None


class DecodeSession:
    """Caches for ``batch`` sequences of up to ``max_len`` tokens, attached to the model's attention layers."""

    def __init__(self, model: nn.Module, batch: int, max_len: int, dtype: torch.dtype | None = None):
        self.model = unwrap(model)
        self.attn = _attention_modules(self.model)
        assert self.attn, "model has no cache-capable attention layers"
        p = next(self.model.parameters())
        self.device, self.dtype = p.device, dtype or p.dtype
        self.batch, self.max_len = int(batch), int(max_len)
        self.seq_lens = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.filled = False
        sms = 148
        a0 = self.attn[0]
        ctas = max(1, batch * a0.n_kv_head)
        # enough CTAs for about four full waves (three resident per SM), but at least two 64-token tiles per split
        self.n_splits = max(1, min(32, (12 * sms + ctas - 1) // ctas, (max_len + 127) // 128))
        self.layers = []
        for a in self.attn:
            # stored head-major ([B, Hk, T, hd]: one contiguous stream per (sequence, head)), used as [B, T, Hk, hd]
            shape = (batch, a.n_kv_head, max_len, a.head_dim)
            self.layers.append(LayerKV(self, torch.zeros(shape, dtype=self.dtype, device=self.device).permute(0, 2, 1, 3),
                                       torch.zeros(shape, dtype=self.dtype, device=self.device).permute(0, 2, 1, 3)))
        self._graph = None
        self._static_ids = None
        self._static_pos = None
        self._static_logits = None

    def __enter__(self) -> "DecodeSession":
        for a, kv in zip(self.attn, self.layers):
            a.kv = kv
        return self

    def __exit__(self, *exc: Any) -> None:
        for a in self.attn:
            a.kv = None
        self._graph = None

    def reset(self) -> None:
        self.seq_lens.zero_()
        self.filled = False

    # ------------------------------------------------------------------ steps
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt ``[B, T]`` (equal lengths) and return the logits of its last position ``[B, V]``."""
        B, T = ids.shape
        assert B == self.batch and T <= self.max_len and not self.filled
        pos = torch.arange(T, device=ids.device)[None, :].expand(B, T)
        hidden = self.model(ids, position_ids=pos, skip_lm_head=True)["hidden"]
        self.seq_lens.fill_(T)
        self.filled = True
        return self.model.head(hidden[:, -1:, :])[:, 0, :]

    def _step_eager(self, ids: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        hidden = self.model(ids, position_ids=pos, skip_lm_head=True)["hidden"]
        return self.model.head(hidden)[:, 0, :]

    @torch.no_grad()
    def step(self, ids: torch.Tensor, use_graph: bool = True) -> torch.Tensor:
        """Append one token per sequence (``ids [B]``) and return the next-token logits ``[B, V]``."""
        assert self.filled, "prefill first"
        if self.device.type != "cuda" or not use_graph:
            self.seq_lens.add_(1)
            pos = (self.seq_lens.to(torch.long) - 1)[:, None]
            return self._step_eager(ids[:, None], pos)
        if self._graph is None:
            self._static_ids = torch.zeros((self.batch, 1), dtype=torch.long, device=self.device)
            self._static_pos = torch.zeros((self.batch, 1), dtype=torch.long, device=self.device)
            keep = self.seq_lens.clone()
            # warm up on a side stream (lazy initialisation must not happen during capture), then capture
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                self._static_ids.copy_(ids[:, None])
                self._advance()
                self._step_eager(self._static_ids, self._static_pos)
                self.seq_lens.copy_(keep)
            torch.cuda.current_stream(self.device).wait_stream(s)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._advance()
                self._static_logits = self._step_eager(self._static_ids, self._static_pos)
            self.seq_lens.copy_(keep)
        self._static_ids.copy_(ids[:, None])
        self._graph.replay()
        return self._static_logits

    def _advance(self) -> None:
        self.seq_lens.add_(1)
        self._static_pos.copy_((self.seq_lens.to(torch.long) - 1)[:, None])


@torch.no_grad()
def generate_stream(model: nn.Module, input_ids: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                    top_k: int | None = None, top_p: float | None = None, greedy: bool = False,
                    eos_token_id: int | None = None, use_kv_cache: bool = True, seed: int = 0,
                    generator: torch.Generator | None = None, use_graph: bool = True) -> Iterator[torch.Tensor]:
    """Yield the new tokens ``[B]`` step by step (finished sequences yield the padding id)."""
    root = unwrap(model)
    is_module = isinstance(root, nn.Module)      # any callable returning {"logits": ...} can be sampled from, uncached
    was_training = root.training if is_module else False
    if is_module:
        root.eval()
    B, T0 = input_ids.shape
    mcfg = getattr(root, "config", None) if is_module else None
    limit = next((int(v) for v in (getattr(mcfg, "sequence_length", None), getattr(mcfg, "block_size", None))
                  if isinstance(v, int) and v > 0), T0 + max_new_tokens)
    pad = eos_token_id if eos_token_id is not None else 0
    finished = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
    pick = lambda lg, i: dec_ops.sample(lg, temperature, top_k, top_p, greedy, seed=seed, offset=i,  # noqa: E731
                                        generator=generator)
    try:
        cached = use_kv_cache and is_module and supports_kv_cache(root) and T0 + max_new_tokens <= limit
        if cached:
            with DecodeSession(root, B, T0 + max_new_tokens) as sess:
                logits = sess.prefill(input_ids)
                for i in range(max_new_tokens):
                    nxt = pick(logits, i)
                    if eos_token_id is not None:
                        nxt = torch.where(finished, torch.full_like(nxt, pad), nxt)
                        finished |= nxt == eos_token_id
                    yield nxt
                    if i + 1 == max_new_tokens or (eos_token_id is not None and bool(finished.all())):
                        break
                    logits = sess.step(nxt, use_graph=use_graph)
        else:
            cur = input_ids
            for i in range(max_new_tokens):
                ctx = cur[:, -limit:]
                logits = model(input_ids=ctx)["logits"][:, -1, :]
                nxt = pick(logits, i)
                if eos_token_id is not None:
                    nxt = torch.where(finished, torch.full_like(nxt, pad), nxt)
                    finished |= nxt == eos_token_id
                yield nxt
                if eos_token_id is not None and bool(finished.all()):
                    break
                cur = torch.cat([cur, nxt[:, None]], dim=1)
    finally:
        if is_module:
            root.train(was_training)


@torch.no_grad()
def generate(model: nn.Module, input_ids: torch.Tensor, max_new_tokens: int, **kwargs: Any) -> torch.Tensor:
    """New tokens ``[B, n]`` (``n <= max_new_tokens``; stops early once every sequence hit EOS)."""
    toks = [t[:, None] for t in generate_stream(model, input_ids, max_new_tokens, **kwargs)]
    if not toks:
        return torch.empty((input_ids.shape[0], 0), dtype=torch.long, device=input_ids.device)
    return torch.cat(toks, dim=1)


@contextlib.contextmanager
def decode_session(model: nn.Module, batch: int, max_len: int):
    with DecodeSession(model, batch, max_len) as s:
        yield s
