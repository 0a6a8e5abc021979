"""Worker: tensor parallel (with sequence parallelism) x sharded data parallel on one mesh, against a
single-process fp32 run on the concatenated batch. Usage: torchrun ... _mp_tp_fsdp_check.py <tp_size>."""
import copy
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.criterion import build_criterion  # noqa: E402
from optimus_dl_b200.model_transforms import build_model_transform  # noqa: E402
from optimus_dl_b200.models import build_model  # noqa: E402
from optimus_dl_b200.ops import _lib  # noqa: E402
from optimus_dl_b200.optim import build_optimizer  # noqa: E402
from optimus_dl_b200.parallel import build_best_collective  # noqa: E402
from optimus_dl_b200.parallel.collective import DistributedConfig  # noqa: E402

CFG = dict(_name="llama2", n_layer=2, n_head=8, n_kv_head=4, n_embd=256, intermediate_size=768, vocab_size=1024,
           sequence_length=256, tie_word_embeddings=False)


def main() -> None:
    tp = int(sys.argv[1]) if len(sys.argv) > 1 else 2
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dp = world // tp
    coll = build_best_collective(DistributedConfig(tp_size=tp, sharding_world_size=dp), dev)
    assert coll.tp_world_size == tp and coll.dp_world_size == dp
    torch.manual_seed(0)
    ref = build_model(CFG)
    gpu = copy.deepcopy(ref).to(dev, torch.bfloat16)
    gpu = build_model_transform({"_name": "tensor_parallel",
                                 "custom_model_kwargs": {"sequence_parallel": True, "loss_parallel": True}}).apply(
        gpu, collective=coll, device=dev)
    gpu = build_model_transform({"_name": "fully_shard"}).apply(gpu, collective=coll, device=dev)
    crit = build_criterion({"_name": "cross_entropy"}, collective=coll)
    opt = build_optimizer({"_name": "adamw", "lr": 1e-3, "betas": [0.9, 0.95], "weight_decay": 0.1},
                          params=gpu.make_parameter_groups())
    groups = ref.make_parameter_groups()
    ref_opt = torch.optim.AdamW([dict(g, params=[p for _, p in g["params"]]) for g in groups], lr=1e-3,
                                betas=(0.9, 0.95), weight_decay=0.1)
    gen = torch.Generator().manual_seed(7)
    ok = True
    for step in range(4):
        ids_all = torch.randint(0, 1024, (dp * 2, 129), generator=gen)
        mine = ids_all[coll.dp_rank * 2:(coll.dp_rank + 1) * 2].to(dev)
        opt.zero_grad()
        loss, _ = crit(gpu, {"input_ids": mine})
        loss.backward()
        opt.step()
        lt = loss.detach().float().clone()
        dist.all_reduce(lt)
        lt /= world
        if rank == 0:
            ref_opt.zero_grad()
            lr_, _ = crit(ref, {"input_ids": ids_all})
            lr_.backward()
            ref_opt.step()
            d = abs(lr_.item() - lt.item())
            print(f"step {step}: ref {lr_.item():.4f} tp{tp}xdp{dp} {lt.item():.4f} diff {d:.4f}", flush=True)
            ok &= d < 6e-2
    torch.cuda.synchronize()
    _lib.check_status(dev)
    if rank == 0:
        print("MP_TP_FSDP_OK" if ok else "MP_TP_FSDP_FAIL", flush=True)
    coll.close()


if __name__ == "__main__":
    main()
