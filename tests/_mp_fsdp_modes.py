"""Worker for test_multigpu.py: the resident and the resharded (reshard_after_forward, pooled slots) modes of the
sharding engine, and every-second-block resharding, must give bitwise equal losses and fp32 master shards: they
run the same kernels on the same values and differ only in where gathered parameters live."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.criterion import build_criterion  # noqa: E402
from optimus_dl_b200.model_transforms import build_model_transform  # noqa: E402
from optimus_dl_b200.model_transforms.distributed import accumulation_context  # noqa: E402
from optimus_dl_b200.models import build_model  # noqa: E402
from optimus_dl_b200.ops import _lib  # noqa: E402
from optimus_dl_b200.optim import build_optimizer  # noqa: E402
from optimus_dl_b200.parallel import build_best_collective  # noqa: E402
from optimus_dl_b200.parallel.collective import DistributedConfig  # noqa: E402


def run(coll, dev, rank, world, fsdp_cfg, model_extra, checkpoint, clip, acc):
    cfg = dict(_name="llama2", n_layer=5, n_head=8, n_kv_head=2, n_embd=256, intermediate_size=768, vocab_size=1024,
               sequence_length=256, tie_word_embeddings=False, **model_extra)
    torch.manual_seed(0)
    model = build_model(cfg).to(dev, torch.bfloat16)
    if checkpoint:
        model = build_model_transform({"_name": "activation_checkpoint", "layer_classes": ["LlamaBlock"]}).apply(
            model, collective=coll, device=dev)
    model = build_model_transform(dict({"_name": "fully_shard"}, **fsdp_cfg)).apply(model, collective=coll, device=dev)
    crit = build_criterion({"_name": "cross_entropy"})
    opt = build_optimizer({"_name": "adamw", "lr": 1e-3, "betas": [0.9, 0.95], "weight_decay": 0.1},
                          params=model.make_parameter_groups())
    if clip > 0:
        opt.set_max_norm(clip)
    gen = torch.Generator().manual_seed(11 + rank)
    losses = []
    crit.grad_scale = 1.0 / acc
    for _ in range(3):
        opt.zero_grad()
        for a in range(acc):
            ids = torch.randint(0, 1024, (2, 129), generator=gen).to(dev)
            with accumulation_context(model, a == acc - 1):
                loss, _ = crit(model, {"input_ids": ids})
                (loss / acc).backward()
        opt.step()
        losses.append(loss.item())
    eng = model._sharding_engine
    eng.verify()
    # one forward pass without a backward (evaluation) goes through the same hooks
    with torch.no_grad():
        ev, _ = crit(model, {"input_ids": torch.randint(0, 1024, (2, 129), generator=gen).to(dev)})
    losses.append(ev.item())
    torch.cuda.synchronize()
    _lib.check_status(dev)
    mem = eng.memory_bytes()
    masters = [g.master.clone() for g in eng.groups]
    del model, opt, eng
    return losses, masters, mem


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    coll = build_best_collective(DistributedConfig(tp_size=1, sharding_world_size=world), dev)
    ok = True
    for clip, acc in ((0.0, 1), (0.7, 2)):
        base = run(coll, dev, rank, world, {}, {}, False, clip, acc)
        variants = {
            "reshard_after_forward": ({"reshard_after_forward": True}, {}, False),
            "three pool slots": ({"reshard_after_forward": True, "param_slots": 3}, {}, False),
            "every second block": ({"reshard_after_forward": True}, {"shard_every_ith_layer": 2}, False),
            "resharded + checkpointing": ({"reshard_after_forward": True}, {}, True),
        }
        for name, (fc, mc, ck) in variants.items():
            got = run(coll, dev, rank, world, fc, mc, ck, clip, acc)
            same = got[0] == base[0] and all(torch.equal(a, b) for a, b in zip(got[1], base[1]))
            flag = torch.tensor([int(same)], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if rank == 0:
                print(f"clip {clip} acc {acc} {name}: losses {got[0]} vs {base[0]} -> {'equal' if flag.item() else 'DIFFERENT'}; "
                      f"slots {got[2]['gathered_parameter_slots']} vs {base[2]['gathered_parameter_slots']} bytes", flush=True)
            ok &= bool(flag.item())
            if name == "reshard_after_forward":
                ok &= got[2]["gathered_parameter_slots"] < base[2]["gathered_parameter_slots"]
    if rank == 0:
        print("MP_MODES_OK" if ok else "MP_MODES_FAIL", flush=True)
    coll.close()


if __name__ == "__main__":
    main()
