"""Next-token cross-entropy (optimus_dl/modules/criterion/cross_entropy.py:33-454).

Batch handling, logged meters and exposed protocols follow the reference:

* with ``labels`` in the batch they are used as given; otherwise ``input_ids`` is shifted
  (``targets = ids[:, 1:]``) and every ``(B, T, ...)`` tensor of the batch loses its last position;
* meters: ``loss``, ``perplexity``, ``accuracy``, ``batch_tokens``, ``total_tokens``, ``batch_samples``,
  ``total_samples``, ``input_max_seq_len``, ``input_mean_seq_len`` (token / sample counts are divided by
  the tensor-parallel size so that the cross-rank sum stays correct);
* protocols on request: ``loss``, ``logits``, ``logits_targets``, ``input_tokens``, ``logits_mask``,
  ``classification``.

When the model offers ``supports_fused_head`` and nobody asked for logits, the head projection,
the loss and their gradients run in the chunked fused kernels of ``ops.cross_entropy`` and full
``[tokens, vocab]`` logits are never built.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F

from ..core.log import warn_once
from ..core.registry import RegistryConfigStrict
from ..metrics.common import cached_lambda, log_averaged, log_averaged_exponent, log_max, log_summed
from ..ops import cross_entropy as ce_ops
from . import register_criterion
from .base import BaseCriterion

LOGIT_PROTOCOLS = {"logits", "logits_targets", "logits_mask", "classification"}


logger = logging.getLogger(__name__)


@dataclass
class CrossEntropyCriterionConfig(RegistryConfigStrict):
    label_smoothing: float = 0.0
    use_liger_kernel: bool | None = None   # accepted for config compatibility; one kernel path exists here
    padding_token_id: int = -100
    logit_softcap: float | None = None
    softcap_type: str = "tanh"
    fused_head: bool | None = None          # None = use the fused linear+CE path whenever it applies
    chunk_rows: int = 4096


@register_criterion("cross_entropy", CrossEntropyCriterionConfig)
class CrossEntropyCriterion(BaseCriterion):
    def __init__(self, cfg, collective: Any = None, **_: Any):
        self.cfg = cfg
        self.collective = collective
        self.label_smoothing = float(cfg.label_smoothing)
        self.padding_token_id = int(cfg.padding_token_id)
        self.softcap = cfg.logit_softcap
        self.softcap_type = cfg.softcap_type
        self.grad_scale = 1.0   # set by the training loop to 1 / accumulation steps

    # ------------------------------------------------------------------ batch preparation
    @staticmethod
    def prepare_batch(batch: dict[str, Any]) -> tuple[dict[str, Any], torch.Tensor]:
        # batches straight from a batcher (no ``to_device`` transform) carry numpy arrays
        batch = {k: (torch.from_numpy(v) if type(v).__module__ == "numpy" and hasattr(v, "dtype") and v.ndim > 0 else v)
                 for k, v in batch.items()}
        if "labels" in batch:
            targets = batch.pop("labels")
            return batch, targets
        ids = batch["input_ids"]
        # the shift below drops one token per ROW; a flat (packed) batch described by cu_seqlens would need one
        # dropped per DOCUMENT, which only the batcher can do (it then supplies ``labels``)
        assert "cu_seqlens" not in batch, "If input is flat, we cannot generate labels and inputs efficiently"
        assert ids.ndim == 2, "Input must be 2D for automatic causal shifting"
        targets = ids[:, 1:]
        T = ids.shape[1]
        out: dict[str, Any] = {}
        for k, v in batch.items():
            if k == "seq_lens" and isinstance(v, torch.Tensor):
                if bool((v < 1).any()):
                    warn_once(logger, "seq_lens contains empty sequences; their shifted length is clamped to 0")
                out[k] = torch.clamp(v - 1, min=0)
            elif isinstance(v, torch.Tensor) and v.dim() >= 2 and v.shape[0] == ids.shape[0] and v.shape[1] == T:
                out[k] = v[:, :-1]
            else:
                out[k] = v
        return out, targets

    def _tp_size(self) -> int:
        return self.collective.tp_world_size if self.collective is not None else 1

    def _log_inputs(self, batch: dict[str, Any]) -> None:
        ids = batch["input_ids"]
        tp = self._tp_size()
        seq_lens = batch.get("seq_lens")
        cu = batch.get("cu_seqlens")
        if cu is not None:
            lens = lambda: (cu[1:] - cu[:-1]).float()  # noqa: E731
            n_samples = lambda: float(cu.numel() - 1)  # noqa: E731
        elif seq_lens is not None:
            lens = lambda: seq_lens.float()  # noqa: E731
            n_samples = lambda: float(seq_lens.numel())  # noqa: E731
        else:
            lens = lambda: torch.full((ids.shape[0],), float(ids.shape[1]))  # noqa: E731
            n_samples = lambda: float(ids.shape[0])  # noqa: E731
        # kinds, weights and rounding as optimus_dl/modules/criterion/cross_entropy.py:133-186 logs them
        log_max("input_max_seq_len", lambda: lens().max().item(), round=2)
        log_averaged("input_mean_seq_len", lambda: lens().mean().item(), weight=lambda: n_samples() / tp, round=2)
        log_summed("batch_samples", lambda: n_samples() / tp)
        log_summed("total_samples", lambda: n_samples() / tp, reset=False)

    # ------------------------------------------------------------------ call
    def __call__(self, model, batch, requested_protocols: set[str] | None = None):
        requested = set(requested_protocols or ())
        batch, targets = self.prepare_batch(batch)
        self._log_inputs(batch)
        targets = targets.contiguous()
        if self.padding_token_id != -100:
            targets = torch.where(targets == self.padding_token_id, torch.full_like(targets, -100), targets)
        flat_targets = targets.reshape(-1)
        want_logits = bool(requested & LOGIT_PROTOCOLS)
        use_fused = self.cfg.fused_head if self.cfg.fused_head is not None else True
        # ``is True``: a stand-in model (unittest.mock.Mock and the like) answers any attribute with a truthy object
        use_fused = use_fused and getattr(model_root(model), "supports_fused_head", False) is True and not want_logits
        exposed: dict[str, Any] = {}
        if use_fused:
            hidden = model(**batch, skip_lm_head=True)["hidden"]
            head_w = model_root(model).lm_head.weight
            tp_group, voff, vtot = head_parallel_info(model_root(model))
            res = ce_ops.linear_cross_entropy(hidden, head_w, flat_targets, ignore_index=-100,
                                              label_smoothing=self.label_smoothing, softcap=self.softcap,
                                              softcap_type=self.softcap_type, chunk_rows=int(self.cfg.chunk_rows),
                                              tp_group=tp_group, vocab_offset=voff, total_vocab=vtot,
                                              grad_scale=self.grad_scale)
            logits = None
        else:
            logits = model(**batch)["logits"]
            res = ce_ops.cross_entropy_ref(logits.reshape(-1, logits.shape[-1]), flat_targets, -100,
                                           self.label_smoothing, self.softcap, self.softcap_type)
        loss = res.loss
        tp = self._tp_size()
        n_valid = cached_lambda(lambda: res.n_valid.item())
        log_averaged("accuracy", lambda: res.n_correct.item() / max(n_valid(), 1), weight=n_valid, round=2)
        log_summed("batch_tokens", lambda: n_valid() / tp)
        log_summed("total_tokens", lambda: n_valid() / tp, reset=False)
        loss_val = cached_lambda(lambda: loss.detach().float().item())
        log_averaged("loss", loss_val, weight=n_valid, priority=0)
        log_averaged_exponent("perplexity", value=loss_val, weight=n_valid, priority=1)
        if "loss" in requested:
            exposed["loss"] = loss.detach()
        if "input_tokens" in requested:
            exposed["input_tokens"] = batch["input_ids"]
        if want_logits and logits is not None:
            lg, tg, mask = self._unflatten(logits, targets, batch)
            if "logits" in requested:
                exposed["logits"] = lg
            if "logits_targets" in requested:
                exposed["logits_targets"] = tg
            if "logits_mask" in requested:
                exposed["logits_mask"] = mask
            if "classification" in requested:
                exposed["classification"] = {"predictions": lg.argmax(-1), "targets": tg, "mask": mask}
        return loss, exposed

    # ------------------------------------------------------------------ helpers of the reference's public surface
    @torch.no_grad()
    def gather_predictions(self, logits: torch.Tensor) -> torch.Tensor:
        """Arg-max token per position (optimus_dl/modules/criterion/cross_entropy.py:410-442). With a
        vocabulary-sharded head (``logits`` holds this rank's slice) the ranks exchange their best value and its
        global index."""
        tp = self._tp_size()
        if tp <= 1 or self.collective is None:
            return logits.argmax(-1)
        tp_world = self.collective.tp_world
        best = logits.max(-1)
        idx = best.indices + self.collective.tp_rank * logits.shape[-1]
        vals = tp_world.all_gather_to_list(best.values)
        idxs = tp_world.all_gather_to_list(idx)
        winner = torch.stack(vals, -1).argmax(-1, keepdim=True)
        return torch.stack(idxs, -1).gather(-1, winner).squeeze(-1)

    @torch.no_grad()
    def accuracy_metric(self, predictions: torch.Tensor, targets: torch.Tensor) -> float:
        """Top-1 accuracy over the valid targets (optimus_dl/modules/criterion/cross_entropy.py:444-454)."""
        valid = (targets >= 0) & (targets != self.padding_token_id)
        correct = ((predictions == targets) & valid).float()
        return (correct.sum() / valid.sum()).item()

    @staticmethod
    def _unflatten(logits: torch.Tensor, targets: torch.Tensor, batch: dict[str, Any]):
        """Packed ``(1, sum T)`` batches are scattered back to ``(docs, max_len)``; others pass through."""
        cu = batch.get("cu_seqlens")
        mask = targets != -100
        if cu is None or logits.shape[0] != 1:
            return logits, targets, mask
        lens = (cu[1:] - cu[:-1]).tolist()
        n, mx = len(lens), max(lens) if lens else 0
        lg = logits.new_zeros((n, mx, logits.shape[-1]))
        tg = targets.new_full((n, mx), -100)
        for i, (s, ln) in enumerate(zip(cu[:-1].tolist(), lens)):
            lg[i, :ln] = logits[0, s:s + ln]
            tg[i, :ln] = targets[0, s:s + ln]
        return lg, tg, tg != -100


def model_root(model: torch.nn.Module) -> torch.nn.Module:
    """Unwrap DDP / checkpoint style wrappers down to the model that owns ``lm_head``."""
    m = model
    for _ in range(4):
        if hasattr(m, "lm_head"):
            return m
        inner = getattr(m, "module", None)
        if inner is None:
            break
        m = inner
    return m


def head_parallel_info(model: torch.nn.Module):
    """``(tp_group, vocab_offset, total_vocab)`` of a vocabulary-sharded head, or ``(None, 0, None)``."""
    info = getattr(model, "_vocab_parallel", None)
    if info is None:
        return None, 0, None
    return info["group"], info["offset"], info["total"]
