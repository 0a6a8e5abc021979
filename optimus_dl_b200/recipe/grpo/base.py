"""GRPO (group-relative policy optimisation) recipe.

One step: sample ``group_size`` completions for each prompt with the KV-cache decoder
(``recipe/generation.py``), score them with a reward function, normalise rewards inside each group,
evaluate sampling-time and frozen-reference log-probabilities with teacher-forced forwards, then do
``updates_per_rollout`` optimizer steps on the clipped-ratio objective with a KL penalty
(``loss.py``). The head projection, the log-probabilities and their gradients run in the chunked
fused kernels (``ops.cross_entropy.linear_token_loss``), so ``[tokens, vocab]`` logits are never
stored. Data parallelism and sharding come from the usual model transforms (``fully_shard``): every
rank rolls out and trains on its own slice of the prompts.

The reference has no RL recipe; builders, loggers, checkpoints and the optimizer step are shared
with the train recipe (optimus_dl/recipe/train/base.py), so the run directory looks the same.
"""

from __future__ import annotations

import logging
import time
from typing import Any

import torch

from ...checkpoint import build_checkpoint_manager
from ...core import conf
from ...core.device import setup_device_and_collective
from ...core.log import setup_logging, trange
from ...core.seed import set_seed
from ...loggers.base import RunStatus
from ...metrics.base import compute_meters, meters_group, reset_meters, step_meters
from ...metrics.common import log_averaged, log_summed
from ...model_transforms.distributed import accumulation_context
from ...models import build_model
from ...ops import cross_entropy as ce_ops
from ..generation import generate, unwrap
from ..mixins.model_builder import build_model_builder
from ..train.builders.optimizer_builder import build_optimizer_builder
from ..train.builders.scheduler_builder import build_scheduler_builder
from ..train.mixins.execution.iteration_mixin import TrainingIterationMixin
from ..train.mixins.managers.logger_manager import build_logger_manager
from .loss import group_advantages, token_loss
from .rewards import build_prompts, build_reward

logger = logging.getLogger(__name__)


class GRPORecipe(TrainingIterationMixin):
    def __init__(self, cfg: Any, **kwargs: Any):
        self.cfg = cfg
        c = cfg.common
        self.output_path = str(c.output_path)
        self.model_builder = build_model_builder(cfg.model_builder, model_transforms=cfg.model_transforms)
        self.optimizer_builder = build_optimizer_builder(cfg.optimizer_builder, optimization_config=cfg.optimization)
        self.scheduler_builder = build_scheduler_builder(cfg.scheduler_builder, lr_scheduler_config=cfg.lr_scheduler,
                                                         optimization_config=cfg.optimization)
        self.logger_manager = build_logger_manager(cfg.logger_manager, loggers_config=cfg.loggers)
        self.checkpoint_manager = build_checkpoint_manager(cfg.checkpoint_manager, output_path=self.output_path)
        self.model = self.ref_model = self.optimizer = None
        self.history: list[dict[str, float]] = []

    # ------------------------------------------------------------------ pieces
    def _build_models(self, device: torch.device, collective: Any):
        g = self.cfg.grpo
        seed = int(self.cfg.common.seed)
        ref = None
        if float(g.kl_coef) > 0:
            # same seed and construction path as the policy => identical initial weights, kept frozen
            set_seed(seed)
            ref = self._plain_model(device)
            for p in ref.parameters():
                p.requires_grad_(False)
            ref.eval()
        set_seed(seed)
        policy = self.model_builder.build_model(self.cfg.model, collective=collective, device=device)
        if getattr(policy, "_sharding_engine", None) is None:
            policy = policy.to(device)
            if device.type == "cuda":
                policy = policy.to(torch.bfloat16)
        return policy, ref

    def _plain_model(self, device: torch.device) -> torch.nn.Module:
        if device.type == "cuda":
            prev = torch.get_default_dtype()
            torch.set_default_dtype(torch.bfloat16)
            try:
                with torch.device(device):
                    return build_model(self.cfg.model)
            finally:
                torch.set_default_dtype(prev)
        return build_model(self.cfg.model).to(device)

    @torch.no_grad()
    def rollout(self, model: torch.nn.Module, prompts: torch.Tensor, step: int) -> tuple[torch.Tensor, torch.Tensor]:
        """``prompts [P, L]`` -> sequences ``[P * G, L + n]`` and the mask ``[P * G, n]`` of tokens that count."""
        g = self.cfg.grpo
        eng = getattr(unwrap(model), "_sharding_engine", None)
        if eng is not None:
            eng.gather_all()
        rep = prompts.repeat_interleave(int(g.group_size), dim=0)
        outs = []
        bs = max(int(g.rollout_batch_size), 1)
        for s in range(0, rep.shape[0], bs):
            chunk = rep[s:s + bs]
            new = generate(model, chunk, int(g.max_new_tokens), temperature=float(g.temperature), top_k=g.get("top_k"),
                           top_p=g.get("top_p"), eos_token_id=g.get("eos_token_id"), use_kv_cache=bool(g.use_kv_cache),
                           seed=int(self.cfg.common.seed) * 7919 + step * 131 + s, use_graph=bool(g.use_cuda_graph))
            if new.shape[1] < int(g.max_new_tokens):  # every sequence of the chunk ended early
                pad = torch.full((new.shape[0], int(g.max_new_tokens) - new.shape[1]), int(g.eos_token_id or 0),
                                 dtype=new.dtype, device=new.device)
                new = torch.cat([new, pad], dim=1)
            outs.append(new)
        completions = torch.cat(outs, dim=0)
        mask = torch.ones_like(completions, dtype=torch.bool)
        eos = g.get("eos_token_id")
        if eos is not None:
            ended = (completions == int(eos)).int().cumsum(-1)
            mask = (ended - (completions == int(eos)).int()) == 0   # keep tokens up to and including the first EOS
        return torch.cat([rep, completions], dim=1), mask

    @torch.no_grad()
    def token_logprobs(self, model: torch.nn.Module, seqs: torch.Tensor, prompt_len: int) -> torch.Tensor:
        """Log-probabilities ``[N, n]`` of the generated tokens under ``model`` (teacher forcing, no gradient)."""
        root = unwrap(model)
        was = root.training
        root.eval()
        mb = max(int(self.cfg.grpo.micro_batch_size), 1)
        out = []
        try:
            for s in range(0, seqs.shape[0], mb):
                x = seqs[s:s + mb]
                hidden = model(x[:, :-1], skip_lm_head=True)["hidden"][:, prompt_len - 1:]
                tg = x[:, prompt_len:]
                _, nll = ce_ops.linear_token_loss(hidden.reshape(-1, hidden.shape[-1]), root.lm_head.weight, tg.reshape(-1),
                                                  lambda n, a, b: (torch.zeros_like(n), torch.zeros_like(n)))
                out.append(-nll.view(tg.shape))
        finally:
            root.train(was)
        return torch.cat(out, dim=0)

    def train_on_rollout(self, model, optimizer, seqs, mask, adv, old_logp, ref_logp, prompt_len: int) -> dict:
        g = self.cfg.grpo
        root = unwrap(model)
        mb = max(int(g.micro_batch_size), 1)
        n_tok = float(mask.sum().clamp(min=1))
        sums = {"loss": 0.0, "kl_sum": 0.0, "clipped_sum": 0.0, "ratio_sum": 0.0}
        optimizer.zero_grad()
        model.train()
        starts = list(range(0, seqs.shape[0], mb))
        for i, s in enumerate(starts):
            x = seqs[s:s + mb]
            tg = x[:, prompt_len:].reshape(-1)
            o = old_logp[s:s + mb].reshape(-1)
            r = ref_logp[s:s + mb].reshape(-1) if ref_logp is not None else None
            a = adv[s:s + mb, None].expand(-1, mask.shape[1]).reshape(-1)
            m = mask[s:s + mb].reshape(-1)
            stats_box: list[dict] = []

            def loss_fn(nll, r0, r1, o=o, r=r, a=a, m=m, stats_box=stats_box):
                lo, d, st = token_loss(nll, o[r0:r1], None if r is None else r[r0:r1], a[r0:r1], m[r0:r1],
                                       float(g.clip_eps), float(g.kl_coef), 1.0 / n_tok)
                stats_box.append(st)
                return lo, d

            with accumulation_context(model, i == len(starts) - 1):
                hidden = model(x[:, :-1], skip_lm_head=True)["hidden"][:, prompt_len - 1:]
                loss, _ = ce_ops.linear_token_loss(hidden.reshape(-1, hidden.shape[-1]), root.lm_head.weight, tg, loss_fn)
                loss.backward()
            sums["loss"] += float(loss.detach())
            for st in stats_box:
                for k in ("kl_sum", "clipped_sum", "ratio_sum"):
                    sums[k] += float(st[k])
        self._optimizer_step(model, optimizer, None, self.cfg.optimization.get("clip_grad_norm"))
        optimizer.zero_grad()
        return {"loss": sums["loss"], "kl": sums["kl_sum"] / n_tok, "clip_frac": sums["clipped_sum"] / n_tok,
                "ratio": sums["ratio_sum"] / n_tok}

    # ------------------------------------------------------------------ run
    def run(self) -> None:
        cfg, c, g = self.cfg, self.cfg.common, self.cfg.grpo
        set_seed(int(c.seed))
        setup = setup_device_and_collective(use_gpu=bool(c.use_gpu), config=c.distributed)
        device, collective = setup.device, setup.collective
        setup_logging(log_path=f"{self.output_path}/logging/rank_{collective.rank}")
        dp_rank, dp_world = collective.dp_rank, collective.dp_world_size
        assert int(g.num_prompts) % dp_world == 0, "num_prompts must be divisible by the data-parallel size"
        n_local = int(g.num_prompts) // dp_world
        model, ref = self._build_models(device, collective)
        optimizer = self.optimizer_builder.build_optimizer(model.make_parameter_groups())
        lr_scheduler = self.scheduler_builder.build_lr_scheduler(optimizer)
        reward_fn = build_reward(g.reward)
        vocab = int(unwrap(model).config.vocab_size)
        prompt_src = build_prompts(g.prompts, vocab_size=vocab, seed=int(c.data_seed), rank=dp_rank, world_size=dp_world)
        self.model, self.ref_model, self.optimizer = model, ref, optimizer
        start, _ = self.checkpoint_manager.load_checkpoint_if_exists(model=model, optimizer=optimizer,
                                                                     lr_scheduler=lr_scheduler, collective=collective,
                                                                     logger_manager=self.logger_manager)
        if collective.is_master:
            self.logger_manager.build_loggers()
            self.logger_manager.setup_loggers(str(c.exp_name), conf.to_container(cfg, resolve=True))
        status = RunStatus.FINISHED
        L = int(g.prompt_length)
        try:
            for it in trange(start, int(cfg.optimization.iterations) + 1, desc="grpo", disable=not collective.is_master):
                with meters_group("train", log_freq=int(c.log_freq)) as should_log:
                    t0 = time.perf_counter()
                    prompts = prompt_src(it, n_local, L, device)
                    seqs, mask = self.rollout(model, prompts, it)
                    if device.type == "cuda":
                        torch.cuda.synchronize(device)
                    t_roll = time.perf_counter() - t0
                    rewards = reward_fn(seqs[:, :L], seqs[:, L:], mask)
                    adv = group_advantages(rewards, int(g.group_size), float(g.advantage_eps))
                    old_logp = self.token_logprobs(model, seqs, L)
                    ref_logp = self.token_logprobs(ref, seqs, L) if ref is not None else None
                    stats = {}
                    for _ in range(max(int(g.updates_per_rollout), 1)):
                        stats = self.train_on_rollout(model, optimizer, seqs, mask, adv, old_logp, ref_logp, L)
                    if lr_scheduler is not None:
                        lr_scheduler.step()
                    if device.type == "cuda":
                        torch.cuda.synchronize(device)
                    t_all = time.perf_counter() - t0
                    n_gen = float(mask.sum())
                    log_averaged("reward", float(rewards.mean()), round=5, priority=0)
                    log_averaged("reward_std", float(rewards.std(unbiased=False)), round=5)
                    log_averaged("loss", stats["loss"], round=6)
                    log_averaged("kl", stats["kl"], round=6)
                    log_averaged("clip_frac", stats["clip_frac"], round=5)
                    log_averaged("ratio", stats["ratio"], round=5)
                    log_summed("generated_tokens", n_gen)
                    log_averaged("perf/rollout_s", t_roll, round=3)
                    log_averaged("perf/step_s", t_all, round=3)
                    log_averaged("perf/rollout_tokens_per_s", n_gen / max(t_roll, 1e-9), round=1)
                    log_averaged("learning_rate", optimizer.param_groups[0]["lr"])
                if should_log:
                    metrics = compute_meters("train", aggregate=True, collective=collective)
                    self.history.append({k: v for k, v in metrics.items() if isinstance(v, (int, float))})
                    if collective.is_master:
                        self.logger_manager.log_metrics_to_loggers(metrics, it, "train")
                        logger.info("iteration %d: %s", it, {k: metrics.get(k) for k in ("reward", "loss", "kl", "clip_frac")})
                step_meters("train")
                if should_log:
                    reset_meters("train")
                persistent = bool(c.save_freq) and it % int(c.save_freq) == 0
                last = bool(c.last_save_freq) and it % int(c.last_save_freq) == 0
                if persistent or last:
                    self.checkpoint_manager.save_checkpoint(
                        iteration=it, model=model, optimizer=optimizer, lr_scheduler=lr_scheduler, collective=collective,
                        full_config=conf.to_container(cfg, resolve=True), persistent=persistent,
                        logger_manager=self.logger_manager)
        except KeyboardInterrupt:
            status = RunStatus.INTERRUPTED
        except Exception:
            status = RunStatus.FAILED
            raise
        finally:
            if collective.is_master:
                self.logger_manager.finished(status)
                self.logger_manager.close_loggers()
            try:
                collective.close()
            except Exception as err:  # noqa: BLE001
                logger.debug("collective.close: %s", err)
