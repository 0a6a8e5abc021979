"""Flagship benchmark: Llama-3-8B bf16 training throughput (tokens/s) under this framework's
fully-sharded engine, on N GPUs of one node.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29501 bench.py --gpus 8 --steps 8 --warmup 3

Prints ONE JSON line (rank 0). ``value`` is device-timed (CUDA events bracketed by a barrier and a
synchronize, max over ranks) over exactly ``--steps`` optimizer steps, each a full forward,
backward, gradient reduce-scatter and sharded AdamW update of the named model on synthetic
uniform-random token ids with random-init weights. ``e2e`` repeats the measurement through the
same public calls a training script makes, adding the per-step host->device copy of the batch from
pinned memory and the device->host read of the loss. ``--impl reference`` runs the unmodified
reference framework on the same config (baseline/reference_arm.py) and prints the same keys.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

MODELS = {
    "llama3-8b": dict(_name="llama2", n_layer=32, n_head=32, n_kv_head=8, n_embd=4096, intermediate_size=14336,
                      vocab_size=128256, rope_theta=500000.0, sequence_length=8192, tie_word_embeddings=False,
                      rmsnorm_eps=1e-5),
    "llama-1b": dict(_name="llama2", n_layer=16, n_head=32, n_kv_head=8, n_embd=2048, intermediate_size=8192,
                     vocab_size=128256, rope_theta=500000.0, sequence_length=8192, tie_word_embeddings=False),
    # BASELINE config 3: Qwen-style 14B (per-head QK-norm), meant for --tp 8 --seq-len 16384 --packed-docs
    "qwen3-14b": dict(_name="qwen3", n_layer=40, n_head=40, n_kv_head=8, n_embd=5120, head_dim=128, intermediate_size=17408,
                      vocab_size=151936, rope_theta=1000000.0, sequence_length=16384, tie_word_embeddings=False,
                      attention_bias=False),
    "tiny": dict(_name="llama2", n_layer=2, n_head=8, n_kv_head=2, n_embd=512, intermediate_size=1536,
                 vocab_size=32000, rope_theta=500000.0, sequence_length=2048, tie_word_embeddings=False),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="llama3-8b", choices=sorted(MODELS))
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (with sequence parallelism and the sharded "
                                                      "loss); the remaining ranks form the sharded data-parallel group")
    ap.add_argument("--fp8", action="store_true", help="e4m3 GEMMs for the transformer blocks' linear layers")
    ap.add_argument("--fp8-recipe", default="blockwise", choices=["blockwise", "tensorwise", "delayed"],
                    help="scaling scheme of --fp8 (1x128 / 128x128 blocks, per tensor, per tensor from a history)")
    ap.add_argument("--acc-steps", type=int, default=1, help="micro-batches accumulated per optimizer step")
    ap.add_argument("--packed-docs", action="store_true", help="each sequence is packed from documents with exponential "
                    "lengths (mean 2048, min 32) and attends block-diagonally")
    ap.add_argument("--timeline", default=None, help="write a per-launcher device-time breakdown of one extra step "
                                                       "(JSON lines) to this file")
    ap.add_argument("--reshard", action="store_true", help="reshard_after_forward: gathered block parameters live in a "
                    "small pool and are gathered again for the backward pass (the memory mode for models that do not fit)")
    ap.add_argument("--n-layer", type=int, default=None, help="override the layer count (profiling only; the "
                    "reported metric then says so)")
    ap.add_argument("--ref-variant", default=None, help="reference arm only: comma-separated list tried in order, from "
                    "'stock' and 'stock+activation_checkpoint' (default: stock, then on one GPU the checkpointed form if "
                    "the stock form runs out of device memory)")
    ap.add_argument("--ref-no-compile", action="store_true", help="reference arm only: leave out the reference's `compile` "
                    "transform (torch.compile of the whole model, which configs/train/train_llama.yaml lists and the arm "
                    "applies by default, falling back to eager execution if compilation fails)")
    args = ap.parse_args()

    if args.impl == "reference":
        # the unmodified reference, in this process, with none of this package imported (baseline/reference_arm.py)
        import importlib.util

        spec = importlib.util.spec_from_file_location(
            "_reference_arm", os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "reference_arm.py"))
        arm = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(arm)
        arm.run(args, MODELS, ClockSampler)
        return

    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.model_transforms import build_model_transform
    from optimus_dl_b200.models import build_model
    from optimus_dl_b200.optim import build_optimizer
    from optimus_dl_b200.ops import _lib
    from optimus_dl_b200.parallel import build_best_collective

    warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}; using WORLD_SIZE", file=sys.stderr)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    from optimus_dl_b200.parallel.collective import DistributedConfig

    tp = max(int(args.tp), 1)
    assert world % tp == 0, "--tp must divide the number of ranks"
    dp = world // tp
    collective = build_best_collective(DistributedConfig(tp_size=tp, sharding_world_size=dp), device)

    mcfg = dict(MODELS[args.model])
    seq = args.seq_len or mcfg["sequence_length"]
    mcfg["sequence_length"] = max(seq, mcfg["sequence_length"])
    if args.n_layer is not None:
        mcfg["n_layer"] = args.n_layer
    torch.manual_seed(0)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(device):
        model = build_model(mcfg)
    torch.set_default_dtype(prev)
    if args.fp8:
        model = build_model_transform({"_name": "transformer_engine", "replace_norm": True}).apply(model)
    if tp > 1:
        model = build_model_transform({"_name": "tensor_parallel", "custom_model_kwargs": {
            "sequence_parallel": True, "loss_parallel": True}}).apply(model, collective=collective, device=device)
    if tp == 1 or dp > 1:
        model = build_model_transform({"_name": "fully_shard", "reshard_after_forward": bool(args.reshard)}).apply(
            model, collective=collective, device=device)
    criterion = build_criterion({"_name": "cross_entropy"}, collective=collective)
    optimizer = build_optimizer({"_name": "adamw", "lr": 3e-4, "betas": [0.9, 0.95], "weight_decay": 0.1},
                                params=model.make_parameter_groups())
    model.train()
    vocab = mcfg["vocab_size"]
    mb = args.micro_batch
    total_steps = warmup + args.steps
    gen = torch.Generator().manual_seed(1234 + collective.dp_rank)   # tensor-parallel peers see the same batch
    acc = max(int(args.acc_steps), 1)
    host_batches = torch.randint(0, vocab, (total_steps, mb * acc, seq + 1), generator=gen, dtype=torch.int64).pin_memory()
    dev_batches = host_batches.to(device)
    doc_ids = None
    if args.packed_docs:
        g2 = torch.Generator().manual_seed(0)
        rows = []
        for _ in range(mb):
            lens, total = [], 0
            while total < seq + 1:
                n = max(32, int(torch.empty(1).exponential_(1.0 / 2048.0, generator=g2).item()))
                lens.append(min(n, seq + 1 - total))
                total += lens[-1]
            rows.append(torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)))
        doc_ids = torch.stack(rows).to(device)

    from optimus_dl_b200.model_transforms.distributed import accumulation_context

    criterion.grad_scale = 1.0 / acc

    import contextlib

    from optimus_dl_b200.amp.fp8 import FP8Recipe, Fp8Format, parse_fp8_recipe

    fp8_recipe = FP8Recipe(Fp8Format.E4M3, parse_fp8_recipe(args.fp8_recipe)) if args.fp8 else None

    def train_step(ids: torch.Tensor) -> torch.Tensor:
        # the backward context is the autocast context plus the delayed-scaling history update on exit
        with (fp8_recipe.backward(True) if fp8_recipe is not None else contextlib.nullcontext()):
            return _train_step(ids)

    def _train_step(ids: torch.Tensor) -> torch.Tensor:
        optimizer.zero_grad()
        loss = None
        for a in range(acc):
            batch = {"input_ids": ids[a * mb:(a + 1) * mb]}
            if doc_ids is not None:
                batch["document_ids"] = doc_ids
            with accumulation_context(model, a == acc - 1):
                loss, _ = criterion(model, batch)
                (loss / acc).backward()
        optimizer.step()
        return loss

    def sync_all() -> None:
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(device)

    def timed(run_step) -> tuple[float, int]:
        for i in range(warmup):
            run_step(i)
        sync_all()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        calls0 = _lib.launch_count()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(warmup, total_steps):
            run_step(i)
        e.record()
        sync_all()
        ms = s.elapsed_time(e)
        launches = _lib.launch_count() - calls0
        clocks = sampler.stop() if rank == 0 else {}
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        _lib.check_status(device)
        return float(t.item()), launches, clocks

    last_loss = {}

    def step_device(i: int) -> None:
        last_loss["v"] = train_step(dev_batches[i])

    def step_e2e(i: int) -> None:
        ids = host_batches[i].to(device, non_blocking=True)
        last_loss["f"] = float(train_step(ids).item())

    ms, launches, clocks = timed(step_device)
    tokens_per_step = dp * mb * acc * seq
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e = None
    if not args.no_e2e:
        ms2, _, _ = timed(step_e2e)
        e2e = {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(host_batches[0].numel() * host_batches.element_size()),
               "d2h_bytes_per_step": 4, "ms_per_step": ms2 / args.steps, "final_loss": last_loss.get("f")}
    if args.timeline and rank == 0:
        # one more step with every launcher call bracketed by CUDA events: per-kernel device time of a step
        # (diagnostics only; the numbers above were measured without it)
        _lib.timeline_start()
        step_device(total_steps - 1)
        report = _lib.timeline_report()
        total = sum(ms_ for _, ms_ in report.values()) or 1.0
        rows = sorted(report.items(), key=lambda kv: -kv[1][1])
        with open(args.timeline, "w") as f:
            for name, (n, ms_) in rows:
                f.write(json.dumps({"launcher": name, "calls": n, "ms": round(ms_, 3), "share": round(ms_ / total, 4)}) + "\n")
    elif args.timeline:
        step_device(total_steps - 1)   # keep the ranks in lockstep for the collectives of that extra step
    if rank == 0:
        out = {
            "metric": "Llama-3-8B FSDP2 bf16 train tokens/s (device-timed, max/rank)"
            if (args.model == "llama3-8b" and args.n_layer is None and tp == 1 and not args.fp8 and not args.reshard)
            else (f"{args.model}{'' if args.n_layer is None else f' ({args.n_layer} layers)'} "
                  f"{'tp' + str(tp) + '+sp x fsdp' + str(dp) if tp > 1 else 'fsdp' + str(dp)}"
                  f"{' resharded' if args.reshard else ''} {'fp8 ' + args.fp8_recipe if args.fp8 else 'bf16'} "
                  "train tokens/s (device-timed, max/rank)"),
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": f"fp8 e4m3 {args.fp8_recipe} GEMMs, bf16 elsewhere" if args.fp8 else "bf16",
            "data": "synthetic uniform-random token ids, random-init weights",
            "impl": "ours",
            "config": {"model": args.model, "global_batch": dp * mb * acc, "seq_len": seq,
                       "parallelism": (f"tp{tp}+sp x fsdp{dp}" if tp > 1 else
                                       (f"fsdp{world}" if world > 1 else "fsdp1 (single GPU, same sharded engine)")),
                       "packed_docs": bool(args.packed_docs),
                       "optimizer": "AdamW fp32 master/moments, fused into the gradient reduce kernel",
                       "l2": "working set (16 GB bf16 weights + activations) far exceeds the 126 MB L2"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "final_loss": float(last_loss["v"].item()) if "v" in last_loss else None,
            "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 2**30,
        }
        eng = getattr(model, "_sharding_engine", None)
        if eng is not None:
            mem = eng.memory_bytes()
            out["engine_memory_gb"] = {k: round(v / 2**30, 3) for k, v in mem.items() if not k.startswith("_")}
            # symmetric allocations (shards, gradient slots) do not go through the caching allocator's statistics
            symmetric = (mem["bf16_shards"] + mem["gradient_slots"]) if world > 1 else 0
            out["peak_mem_incl_symmetric_gb"] = out["peak_mem_gb"] + symmetric / 2**30
        print(json.dumps(out))
    if world > 1:
        collective.close()


if __name__ == "__main__":
    main()
