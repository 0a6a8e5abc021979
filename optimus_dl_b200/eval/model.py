"""Adapter that lets the ``lm_eval`` harness drive a model of this package
(optimus_dl/modules/eval/model.py:14-242).

Implements the harness's three request kinds. ``loglikelihood`` and ``loglikelihood_rolling`` score
with one forward per *batch* of requests (right-padded, the padded positions are masked out of the
sums); ``generate_until`` decodes greedily with the KV cache and stops at the first stop string.
The class derives from ``lm_eval.api.model.LM`` when the harness is installed and is a plain object
otherwise, so it can be unit-tested without it.
"""

from __future__ import annotations

import logging
from typing import Any

import torch

from ..recipe.generation import generate_stream, unwrap

logger = logging.getLogger(__name__)

try:  # pragma: no cover - depends on the environment
    from lm_eval.api.model import LM as _LMBase
except Exception:  # noqa: BLE001
    class _LMBase:  # type: ignore[no-redef]
        def __init__(self) -> None:
            pass


def _args(request: Any) -> tuple:
    return tuple(request.args) if hasattr(request, "args") else tuple(request)


class LLMBaselinesModel(_LMBase):
    def __init__(self, model: torch.nn.Module, tokenizer: Any, tokenizer_config: Any = None,
                 device: torch.device | str = "cpu", batch_size: int = 8, max_gen_toks: int = 256,
                 reference_scoring: bool = False):
        """``reference_scoring``: score exactly as optimus_dl/modules/eval/model.py:69-165 does, for numbers that have
        to be compared with runs of the reference: context and continuation are encoded separately WITH the
        tokenizer's special tokens (so a BOS token sits between them), an empty context is left empty, and the
        rolling log-likelihood does not score the first token. The default follows the harness's own conventions
        (special tokens stripped from the pieces, an end-of-text token as the empty context, every token scored,
        windows for texts longer than the model's context)."""
        super().__init__()
        self.reference_scoring = bool(reference_scoring)
        self.model = model.eval()
        self.tokenizer = tokenizer
        self.tokenizer_config = tokenizer_config
        self._device = torch.device(device)
        self.batch_size = max(int(batch_size), 1)
        self.max_gen_toks = int(max_gen_toks)
        cfg = unwrap(model).config
        self.max_length = int(getattr(cfg, "sequence_length", None) or getattr(cfg, "block_size", 1024))

    # ------------------------------------------------------------------ harness properties
    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def eot_token_id(self) -> int:
        eos = getattr(self.tokenizer, "eos_token_id", None)
        return int(eos) if eos is not None else 0

    @property
    def rank(self) -> int:
        return 0

    @property
    def world_size(self) -> int:
        return 1

    def tok_encode(self, text: str) -> list[int]:
        ids = list(self.tokenizer.encode(text))
        bos, eos = getattr(self.tokenizer, "bos_token_id", None), getattr(self.tokenizer, "eos_token_id", None)
        add_bos = getattr(self.tokenizer_config, "add_bos", True) if self.tokenizer_config is not None else True
        add_eos = getattr(self.tokenizer_config, "add_eos", True) if self.tokenizer_config is not None else True
        if add_bos and bos is not None and ids and ids[0] == bos:
            ids = ids[1:]
        if add_eos and eos is not None and ids and ids[-1] == eos:
            ids = ids[:-1]
        return ids

    def tok_decode(self, ids: list[int]) -> str:
        return self.tokenizer.decode(list(ids))

    # ------------------------------------------------------------------ scoring
    @torch.no_grad()
    def _score(self, pairs: list[tuple[list[int], list[int]]]) -> list[tuple[float, bool]]:
        """For each ``(context, continuation)`` token pair: ``(sum log p(continuation | context), is_greedy)``."""
        out: list[tuple[float, bool]] = [(0.0, True)] * len(pairs)
        order = sorted(range(len(pairs)), key=lambda i: -(len(pairs[i][0]) + len(pairs[i][1])))
        for s in range(0, len(order), self.batch_size):
            idx = order[s:s + self.batch_size]
            rows, spans = [], []
            for i in idx:
                ctx, cont = pairs[i]
                full = (ctx + cont)[-(self.max_length + 1):]
                n_cont = min(len(cont), len(full) - 1)
                rows.append(full[:-1])
                spans.append((len(full) - 1 - n_cont, len(full) - 1, full[len(full) - n_cont:]))
            T = max(len(r) for r in rows)
            x = torch.zeros((len(rows), T), dtype=torch.long)
            for j, r in enumerate(rows):
                x[j, : len(r)] = torch.tensor(r, dtype=torch.long)
            seq_lens = torch.tensor([len(r) for r in rows], dtype=torch.long)
            logits = self.model(x.to(self._device), seq_lens=seq_lens.to(self._device))["logits"].float()
            logp = torch.log_softmax(logits, dim=-1).cpu()
            for j, i in enumerate(idx):
                a, b, targets = spans[j]
                if b <= a:
                    out[i] = (0.0, True)
                    continue
                tgt = torch.tensor(targets, dtype=torch.long)
                lp = logp[j, a:b]
                out[i] = (float(lp.gather(-1, tgt[:, None]).sum()), bool((lp.argmax(-1) == tgt).all()))
        return out

    def loglikelihood(self, requests: list) -> list[tuple[float, bool]]:
        pairs = []
        for r in requests:
            context, continuation = _args(r)[:2]
            if self.reference_scoring:
                pairs.append((list(self.tokenizer.encode(context)), list(self.tokenizer.encode(continuation))))
                continue
            ctx = self.tok_encode(context) if context else []
            if not ctx:
                ctx = [self.eot_token_id]
            pairs.append((ctx, self.tok_encode(continuation)))
        return self._score(pairs)

    def loglikelihood_rolling(self, requests: list) -> list[float]:
        res = []
        for r in requests:
            (text,) = _args(r)[:1]
            if self.reference_scoring:
                raw = list(self.tokenizer.encode(text))
                res.append(self._score([(raw[:1], raw[1:])])[0][0] if len(raw) > 1 else 0.0)
                continue
            ids = self.tok_encode(text)
            total, prev = 0.0, [self.eot_token_id]
            # disjoint windows of at most max_length targets, each conditioned on the previous window's tail
            for s in range(0, len(ids), self.max_length):
                chunk = ids[s:s + self.max_length]
                ctx = prev[-1:] if s == 0 else ids[max(0, s - 1):s]
                total += self._score([(ctx, chunk)])[0][0]
            res.append(total)
        return res

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate_until(self, requests: list) -> list[str]:
        outs = []
        for r in requests:
            context, kwargs = _args(r)[:2]
            kwargs = dict(kwargs or {})
            until = kwargs.get("until") or []
            until = [until] if isinstance(until, str) else list(until)
            max_new = int(kwargs.get("max_gen_toks", self.max_gen_toks))
            temperature = float(kwargs.get("temperature", 0.0) or 0.0)
            ids = self.tok_encode(context) or [self.eot_token_id]
            max_new = max(1, min(max_new, self.max_length - 1))
            ids = ids[-(self.max_length - max_new):]
            x = torch.tensor([ids], dtype=torch.long, device=self._device)
            toks: list[int] = []
            text = ""
            for t in generate_stream(self.model, x, max_new, temperature=temperature, greedy=temperature <= 0,
                                     eos_token_id=None):
                tok = int(t[0])
                if tok == self.eot_token_id and getattr(self.tokenizer, "eos_token_id", None) is not None:
                    break
                toks.append(tok)
                text = self.tok_decode(toks)
                if any(u and u in text for u in until):
                    break
            for u in until:
                if u and u in text:
                    text = text.split(u)[0]
            outs.append(text)
        return outs
