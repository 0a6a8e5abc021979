"""Evaluation recipe: run ``lm_eval`` harness tasks on a checkpoint or a freshly built model
(optimus_dl/recipe/eval/base.py:20-158). The harness is an optional dependency; without it
``run()`` raises ``ImportError`` with an install hint while ``build_eval_model`` still works."""

from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Any

import torch

from ...checkpoint import build_checkpoint_manager
from ...core.seed import set_seed
from ...eval import LLMBaselinesModel
from ...models import build_model
from ...tokenizer import build_tokenizer
from .config import validate

logger = logging.getLogger(__name__)


class EvalRecipe:
    def __init__(self, cfg: Any):
        validate(cfg)
        self.cfg = cfg
        self.model: LLMBaselinesModel | None = None
        self.tokenizer = None

    def device(self) -> torch.device:
        return torch.device("cuda" if bool(self.cfg.common.use_gpu) and torch.cuda.is_available() else "cpu")

    def build_eval_model(self, device: torch.device | None = None) -> LLMBaselinesModel:
        if self.model is not None:
            return self.model
        c = self.cfg.common
        ckpt, model_cfg = c.get("checkpoint_path"), c.get("model")
        assert (ckpt is not None) ^ (model_cfg is not None), \
            "Either checkpoint_path or model must be specified, but not both"
        device = device or self.device()
        if ckpt is not None:
            logger.info("loading model from checkpoint %s", ckpt)
            manager = build_checkpoint_manager({"_name": "base"}, output_path=str(ckpt))
            base, _ = manager.build_model_from_checkpoint(str(ckpt), device=device)
        else:
            logger.info("building model from config")
            base = build_model(model_cfg).to(device)
        if device.type == "cuda":
            base = base.to(torch.bfloat16)
        self.tokenizer = build_tokenizer(c.tokenizer)
        self.model = LLMBaselinesModel(base.eval(), self.tokenizer, c.tokenizer, device=device,
                                       batch_size=int(self.cfg.lm_eval.batch_size),
                                       reference_scoring=bool(self.cfg.lm_eval.get("reference_scoring", False)))
        return self.model

    def run_lm_eval(self) -> dict:
        try:
            from lm_eval import evaluator
        except ImportError as err:
            raise ImportError("lm_eval is required for evaluation. Install with: pip install lm_eval") from err
        set_seed(int(self.cfg.common.seed))
        model = self.build_eval_model()
        raw = self.cfg.lm_eval.tasks
        tasks = [raw] if isinstance(raw, str) else [str(t) for t in raw]
        logger.info("running lm_eval on %s (%d-shot)", tasks, int(self.cfg.lm_eval.num_fewshot))
        results = evaluator.simple_evaluate(model=model, tasks=tasks, num_fewshot=int(self.cfg.lm_eval.num_fewshot),
                                            batch_size=int(self.cfg.lm_eval.batch_size), limit=self.cfg.lm_eval.limit,
                                            device=str(model.device), use_cache=None)
        if results is None:
            raise RuntimeError("Evaluation returned no results")
        out = self.cfg.lm_eval.get("output_path")
        if out:
            p = Path(str(out))
            p.parent.mkdir(parents=True, exist_ok=True)
            p.write_text(json.dumps(results, indent=2, default=str))
            logger.info("results saved to %s", p)
        return results

    def run(self) -> dict:
        results = self.run_lm_eval()
        for task, metrics in (results.get("results") or {}).items():
            logger.info("%s: %s", task, {k: v for k, v in metrics.items() if isinstance(v, (int, float))})
        return results
