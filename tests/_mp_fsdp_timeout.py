"""Worker for test_multigpu.py: a rank that does not take part in a step (made on the host: it simply skips the
step, with none of its kernels in flight) makes the other rank's bounded barrier waits run out. That rank's step must
raise and leave its fp32 master weights and moments as they were. No GPU faults, traps or hangs are involved: the
waiting kernels give up after their (here shortened) poll limit and return normally."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_dl_b200.criterion import build_criterion  # noqa: E402
from optimus_dl_b200.model_transforms import build_model_transform  # noqa: E402
from optimus_dl_b200.models import build_model  # noqa: E402
from optimus_dl_b200.ops import _lib  # noqa: E402
from optimus_dl_b200.optim import build_optimizer  # noqa: E402
from optimus_dl_b200.parallel import build_best_collective  # noqa: E402
from optimus_dl_b200.parallel.collective import DistributedConfig  # noqa: E402


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    coll = build_best_collective(DistributedConfig(tp_size=1, sharding_world_size=world), dev)
    cfg = dict(_name="llama2", n_layer=2, n_head=8, n_kv_head=2, n_embd=256, intermediate_size=768, vocab_size=1024,
               sequence_length=256, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = build_model(cfg).to(dev, torch.bfloat16)
    model = build_model_transform({"_name": "fully_shard"}).apply(model, collective=coll, device=dev)
    crit = build_criterion({"_name": "cross_entropy"})
    opt = build_optimizer({"_name": "adamw", "lr": 1e-3}, params=model.make_parameter_groups())
    eng = model._sharding_engine
    ids = torch.randint(0, 1024, (2, 129), device=dev)

    def one_step():
        opt.zero_grad()
        loss, _ = crit(model, {"input_ids": ids})
        loss.backward()
        opt.step()

    for _ in range(2):
        one_step()
    eng.verify()
    eng.host_sync()
    store = torch.distributed.distributed_c10d._get_default_store()
    if rank == 0:
        _lib.set_flag_wait_iters(1 << 16)        # tens of milliseconds per wait instead of two seconds
        masters = [g.master.clone() for g in eng.groups]
        moments = [g.exp_avg_sq.clone() for g in eng.groups]
        raised = False
        try:
            one_step()                            # rank 1 never launches this step: every barrier of it runs out
            eng.verify()
        except _lib.KernelError as e:
            raised = "flag wait timed out" in str(e)
        torch.cuda.synchronize()
        kept = all(torch.equal(a, g.master) for a, g in zip(masters, eng.groups)) and \
            all(torch.equal(a, g.exp_avg_sq) for a, g in zip(moments, eng.groups))
        print(f"raised={raised} state_kept={kept}", flush=True)
        print("MP_TIMEOUT_OK" if raised and kept else "MP_TIMEOUT_FAIL", flush=True)
        store.set("timeout_test_done", "1")
    else:
        # stays alive (its memory is mapped by rank 0) and idle until rank 0 has finished, then both leave
        t0 = time.time()
        while time.time() - t0 < 120:
            try:
                if store.check(["timeout_test_done"]):
                    break
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.2)
    torch.cuda.synchronize()
    os._exit(0)      # no collective teardown: the ranks are deliberately out of step


if __name__ == "__main__":
    main()
