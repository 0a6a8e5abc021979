"""GRPO step benchmark: ``python -m optimus_dl_b200.recipe.grpo.benchmark [--model qwen3-1.7B] [--prompts 8]``
(``torchrun`` for several GPUs). Runs the recipe's own rollout / scoring / update path on synthetic prompts and
prints one JSON line with device-timed phase durations: rollout (prefill + CUDA-graph decode + fused sampler),
teacher-forced log-probabilities (policy and frozen reference), and the optimizer update."""

from __future__ import annotations

import argparse
import json
import os

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-1.7B")
    ap.add_argument("--prompts", type=int, default=8, help="prompts per GPU and step")
    ap.add_argument("--prompt-length", type=int, default=256)
    ap.add_argument("--group-size", type=int, default=8)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    args = ap.parse_args()

    from ...core import conf
    from ...core.config_utils import non_resolving_instantiate
    from ...core.device import setup_device_and_collective
    from ...core.registry import build
    from .loss import group_advantages
    from .rewards import build_prompts, build_reward

    world = int(os.environ.get("WORLD_SIZE", 1))
    cfg = conf.create({
        "_name": "base",
        "common": {"use_gpu": True, "output_path": "/tmp/grpo_bench", "seed": 0,
                   "distributed": {"tp_size": 1, "sharding_world_size": None}},
        "model": {"_name": args.model},
        "model_transforms": [{"_name": "fully_shard"}],
        "grpo": {"num_prompts": args.prompts * world, "prompt_length": args.prompt_length, "group_size": args.group_size,
                 "max_new_tokens": args.new_tokens, "micro_batch_size": args.micro_batch,
                 "rollout_batch_size": args.prompts * args.group_size},
        "optimization": {"iterations": 1, "optimizer": {"_name": "adamw", "lr": 1e-6, "weight_decay": 0.0}},
    })
    recipe = build("grpo_recipe", non_resolving_instantiate(cfg))
    g = recipe.cfg.grpo
    setup = setup_device_and_collective(use_gpu=True, config=recipe.cfg.common.distributed)
    device, collective = setup.device, setup.collective
    model, ref = recipe._build_models(device, collective)
    optimizer = recipe.optimizer_builder.build_optimizer(model.make_parameter_groups())
    reward_fn = build_reward(g.reward)
    src = build_prompts(g.prompts, vocab_size=int(model.config.vocab_size), seed=0, rank=collective.dp_rank,
                        world_size=collective.dp_world_size)
    L = int(g.prompt_length)

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    phases = {"rollout": 0.0, "logprobs": 0.0, "update": 0.0}
    total_steps = args.warmup + args.steps
    for it in range(total_steps):
        prompts = src(it, args.prompts, L, device)
        e0 = ev()
        seqs, mask = recipe.rollout(model, prompts, it)
        e1 = ev()
        rewards = reward_fn(seqs[:, :L], seqs[:, L:], mask)
        adv = group_advantages(rewards, int(g.group_size))
        old = recipe.token_logprobs(model, seqs, L)
        refp = recipe.token_logprobs(ref, seqs, L) if ref is not None else None
        e2 = ev()
        recipe.train_on_rollout(model, optimizer, seqs, mask, adv, old, refp, L)
        e3 = ev()
        torch.cuda.synchronize()
        if it >= args.warmup:
            phases["rollout"] += e0.elapsed_time(e1)
            phases["logprobs"] += e1.elapsed_time(e2)
            phases["update"] += e2.elapsed_time(e3)
    t = torch.tensor([phases["rollout"], phases["logprobs"], phases["update"]], device=device, dtype=torch.float64) / args.steps
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    if collective.is_master:
        n_seq = args.prompts * args.group_size * world
        gen = n_seq * args.new_tokens
        step_ms = float(t.sum())
        print(json.dumps({
            "metric": "GRPO step (rollout + log-probs + update), device-timed, max over ranks", "model": args.model,
            "n_gpus": world, "sequences_per_step": n_seq, "prompt_length": L, "new_tokens": args.new_tokens,
            "rollout_ms": round(float(t[0]), 1), "logprobs_ms": round(float(t[1]), 1), "update_ms": round(float(t[2]), 1),
            "step_ms": round(step_ms, 1), "generated_tokens_per_s_rollout": round(gen / float(t[0]) * 1e3, 1),
            "decode_ms_per_token_step": round(float(t[0]) / args.new_tokens, 3),
            "generated_tokens_per_s_step": round(gen / step_ms * 1e3, 1),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(device) / 2**30, 1)}))
    collective.close()


if __name__ == "__main__":
    main()
