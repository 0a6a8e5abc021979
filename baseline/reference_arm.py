"""Reference arm of bench.py: the unmodified reference framework on the flagship config.

The reference package tree (`optimus_dl/`, byte-identical to the upstream sources) sits under
`baseline/_ref/`; the third-party modules it imports that this image lacks (`omegaconf`, `hydra`,
`colorlog`, `lm_eval`) are served by the small stand-ins under `baseline/ref_deps/`. Everything that is
timed is the reference's own code, reached through its public registries:

* `ModelBuilder.build_model` -> `Llama` (optimus_dl/modules/model/llama2.py:142), Liger RMSNorm / SwiGLU
  where the reference auto-enables them, its attention block (SDPA / flash-attn dispatch);
* `FullyShardTransform` (optimus_dl/modules/model_transforms/distributed.py:212) with
  `reshard_after_forward: false` (configs/train/train_llama.yaml) and the README's mixed-precision
  policy (bf16 parameters, fp32 gradient reduction); on one rank the reference itself skips the wrapping;
* `CrossEntropyCriterion` (optimus_dl/modules/criterion/cross_entropy.py:42);
* `adamw` with `fused=True` (optimus_dl/modules/optim/adamw.py:42);
* bf16 autocast as built by the train recipe (optimus_dl/recipe/train/mixins/execution/context_mixin.py:136);
* the `compile` transform (optimus_dl/modules/model_transforms/compile.py:33) last, as configs/train/train_llama.yaml
  lists it; if `torch.compile` fails on this image the same model runs eagerly and the printed line says which ran.

This module imports nothing from `optimus_dl_b200` and loads none of its native libraries.
The training step, the synthetic data, warm-up, CUDA-event timing and max-over-ranks are the same as in
the framework's own arm in bench.py.
"""

from __future__ import annotations

import gc
import hashlib
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root() -> str | None:
    """Directory holding the reference's `optimus_dl/` package, or None."""
    for root in (os.path.join(HERE, "_ref"), os.environ.get("OPTIMUS_REFERENCE_ROOT", "")):
        if root and os.path.isfile(os.path.join(root, "optimus_dl", "core", "registry.py")):
            return root
    return None


def tree_digest(pkg_dir: str) -> str:
    """sha256 over the relative paths and contents of every .py / .typed file of a package tree."""
    h = hashlib.sha256()
    for base, dirs, files in sorted(os.walk(pkg_dir)):
        dirs[:] = sorted(d for d in dirs if d != "__pycache__")
        for name in sorted(files):
            if name.endswith((".pyc", ".pyo")):
                continue
            p = os.path.join(base, name)
            h.update(os.path.relpath(p, pkg_dir).encode())
            with open(p, "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def ensure_reference_tree(source: str = "/root/reference/optimus_dl") -> bool:
    """Complete `baseline/_ref/optimus_dl` from an upstream checkout when one is reachable (pip installs only the
    top-level `__init__.py` because the upstream pyproject lists no sub-packages). Returns True if the tree is usable."""
    dst = os.path.join(HERE, "_ref", "optimus_dl")
    if os.path.isfile(os.path.join(dst, "core", "registry.py")):
        return True
    if not os.path.isdir(source):
        return False
    import shutil

    os.makedirs(os.path.dirname(dst), exist_ok=True)
    shutil.copytree(source, dst, dirs_exist_ok=True, ignore=shutil.ignore_patterns("__pycache__"))
    return True


def _print_unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))


def run(args, models: dict, clock_sampler_cls) -> None:
    ensure_reference_tree()
    root = reference_root()
    if root is None:
        _print_unavailable("reference package tree not found under baseline/_ref (and no upstream checkout to copy)")
        return
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(HERE, "ref_deps"))
    assert "optimus_dl_b200" not in sys.modules

    import contextlib
    import logging

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        _print_unavailable("no CUDA device on this machine (the reference arm runs on a B200 like the framework's own arm)")
        return
    logging.disable(logging.INFO)
    try:
        import optimus_dl  # noqa: F401  (bootstraps every registry of the reference)
        from optimus_dl.modules.criterion import build_criterion
        from optimus_dl.modules.distributed import build_best_collective
        from optimus_dl.modules.distributed.config import DistributedConfig
        from optimus_dl.modules.optim import build_optimizer
        from optimus_dl.recipe.mixins.model_builder import ModelBuilder, ModelBuilderConfig
    except Exception as e:  # import failure of the reference itself
        _print_unavailable(f"reference does not import here: {type(e).__name__}: {e}"[:300])
        return

    warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("LOCAL_WORLD_SIZE", str(world))
    collective = build_best_collective(DistributedConfig(tp_size=1, sharding_world_size=world), device)

    mcfg = dict(models[args.model])
    seq = args.seq_len or mcfg["sequence_length"]
    mcfg["sequence_length"] = max(seq, mcfg["sequence_length"])
    if args.n_layer is not None:
        mcfg["n_layer"] = args.n_layer
    mb = args.micro_batch
    acc = max(int(args.acc_steps), 1)
    vocab = mcfg["vocab_size"]
    total_steps = warmup + args.steps

    names = [v for v in (args.ref_variant or "").split(",") if v] or (
        ["stock", "stock+activation_checkpoint"] if world == 1 else ["stock"])
    # the reference's own training config lists the `compile` transform after `fully_shard`
    # (configs/train/train_llama.yaml), so that is the form measured first; if torch.compile fails on this image the
    # same variant runs eagerly and the JSON line says so
    compile_modes = [False] if args.ref_no_compile else [True, False]
    variants = [(n, c) for n in names for c in compile_modes]

    def build(variant: str, use_compile: bool):
        transforms = [{"_name": "fully_shard", "reshard_after_forward": False,
                       "mixed_precision": {"param_dtype": "bfloat16", "reduce_dtype": "float32"}}]
        if "activation_checkpoint" in variant:
            transforms.insert(0, {"_name": "activation_checkpoint", "layer_classes": ["LlamaBlock"]})
        if use_compile:
            transforms.append({"_name": "compile"})
        torch.manual_seed(0)
        builder = ModelBuilder(ModelBuilderConfig(), model_transforms=transforms)
        with torch.device(device):   # parameters are created on the GPU: 8 ranks x 32 GB of fp32 would not fit host memory
            model = builder.build_model(dict(mcfg), collective=collective)
        criterion = build_criterion({"_name": "cross_entropy"}, collective=collective)
        optimizer = build_optimizer({"_name": "adamw", "lr": 3e-4, "betas": [0.9, 0.95], "weight_decay": 0.1, "fused": True},
                                    params=model.make_parameter_groups())
        model.train()
        return model, criterion, optimizer

    gen = torch.Generator().manual_seed(1234 + collective.dp_rank)
    host_batches = torch.randint(0, vocab, (total_steps, mb * acc, seq + 1), generator=gen, dtype=torch.int64).pin_memory()
    dev_batches = host_batches.to(device)

    def sync_all() -> None:
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(device)

    result = None
    tried = []
    for variant, use_compile in variants:
        model = criterion = optimizer = None
        try:
            model, criterion, optimizer = build(variant, use_compile)
            amp_ctx = lambda: torch.autocast(device.type, dtype=torch.bfloat16, enabled=True)  # noqa: E731
            accumulation = getattr(model, "accumulation_context", None)

            def train_step(ids):
                optimizer.zero_grad()
                loss = None
                for a in range(acc):
                    batch = {"input_ids": ids[a * mb:(a + 1) * mb]}
                    ctx = accumulation(a == acc - 1) if accumulation is not None else contextlib.nullcontext()
                    with ctx:
                        with amp_ctx():
                            loss, _ = criterion(model, batch)
                        (loss / acc).backward()
                model.pre_optimizer_step() if hasattr(model, "pre_optimizer_step") else None
                optimizer.step()
                model.post_optimizer_step() if hasattr(model, "post_optimizer_step") else None
                return loss

            last = {}

            def timed(run_step):
                for i in range(warmup):
                    run_step(i)
                sync_all()
                sampler = clock_sampler_cls(local_rank)
                if rank == 0:
                    sampler.start()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for i in range(warmup, total_steps):
                    run_step(i)
                e.record()
                sync_all()
                ms = s.elapsed_time(e)
                clocks = sampler.stop() if rank == 0 else {}
                t = torch.tensor([ms], device=device, dtype=torch.float64)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t.item()), clocks

            def step_device(i):
                last["v"] = train_step(dev_batches[i])

            def step_e2e(i):
                ids = host_batches[i].to(device, non_blocking=True)
                last["f"] = float(train_step(ids).item())

            t0 = time.time()
            ms, clocks = timed(step_device)
            tokens_per_step = world * mb * acc * seq
            value = tokens_per_step * args.steps / (ms / 1e3)
            e2e = None
            if not args.no_e2e:
                ms2, _ = timed(step_e2e)
                e2e = {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s",
                       "h2d_bytes_per_step": int(host_batches[0].numel() * host_batches.element_size()),
                       "d2h_bytes_per_step": 4, "ms_per_step": ms2 / args.steps, "final_loss": last.get("f")}
            result = dict(variant=variant, compiled=use_compile, ms=ms, value=value, clocks=clocks, e2e=e2e,
                          final_loss=float(last["v"].item()), wall_s=time.time() - t0)
            break
        except torch.OutOfMemoryError as err:
            tried.append(f"{variant}{' + compile' if use_compile else ''}: out of device memory ({str(err)[:80]})")
            # every rank takes the same branch: memory use is symmetric across ranks
            model = criterion = optimizer = None
            gc.collect()
            torch.cuda.empty_cache()
            continue
        except Exception as err:  # noqa: BLE001
            if not use_compile:
                raise
            tried.append(f"{variant} + compile: {type(err).__name__}: {str(err)[:120]}")
            model = criterion = optimizer = None
            gc.collect()
            torch.cuda.empty_cache()
            if world > 1:
                dist.barrier(device_ids=[local_rank])
            continue

    if rank == 0:
        if result is None:
            print(json.dumps({"impl": "reference", "unavailable": "; ".join(tried)[:400]}))
        else:
            loaded = sorted({os.path.basename(l.split()[-1]) for l in open("/proc/self/maps") if "libob_" in l})
            out = {
                "metric": "Llama-3-8B FSDP2 bf16 train tokens/s (device-timed, max/rank)" if (args.model == "llama3-8b" and args.n_layer is None)
                else f"{args.model} bf16 train tokens/s (device-timed, max/rank)",
                "value": result["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
                "ms_per_step": result["ms"] / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
                "impl": "reference",
                "config": {"model": args.model, "global_batch": world * mb * acc, "seq_len": seq,
                           "parallelism": (f"fsdp{world}" if world > 1 else "single GPU (the reference skips FSDP wrapping on one rank)"),
                           "packed_docs": False,
                           "optimizer": "torch.optim.AdamW(fused=True) on fp32 parameters" + (" sharded by FSDP2" if world > 1 else ""),
                           "reference_variant": result["variant"], "variants_that_failed": tried,
                           "torch_compile": result["compiled"],
                           "precision": ("FSDP2 MixedPrecisionPolicy(param bf16, reduce fp32) + bf16 autocast" if world > 1
                                         else "fp32 parameters + bf16 autocast (the reference's AMP path)"),
                           "reference_tree_sha256": tree_digest(os.path.join(root, "optimus_dl")),
                           "l2": "working set far exceeds the 126 MB L2"},
                "clocks": result["clocks"], "e2e": result["e2e"], "gpu_launches": None,
                "own_native_libraries_loaded": loaded,
                "final_loss": result["final_loss"],
                "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 2**30,
            }
            print(json.dumps(out))
    if world > 1:
        collective.close()
