"""Worker: the ``ddp`` transform on two Gloo ranks reproduces a single process that sees both ranks' data,
with and without gradient accumulation. Run under torchrun-style environment variables."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def main() -> None:
    from optimus_dl_b200.model_transforms import build_model_transform
    from optimus_dl_b200.model_transforms.distributed import accumulation_context
    from optimus_dl_b200.models import build_model
    from optimus_dl_b200.parallel.collective import build_best_collective

    coll = build_best_collective(device=torch.device("cpu"))
    rank, world = coll.rank, coll.world_size
    assert world == 2 and coll.dp_world_size == 2 and coll.tp_world_size == 1
    cfg = dict(_name="llama2", n_layer=1, n_head=2, n_kv_head=1, n_embd=32, vocab_size=61, sequence_length=16, multiple_of=8)
    torch.manual_seed(0)
    ref = build_model(cfg)
    torch.manual_seed(0)
    model = build_model(cfg)
    ddp = build_model_transform({"_name": "ddp"}).apply(model, collective=coll, device=torch.device("cpu"))
    assert ddp.make_parameter_groups()                            # BaseModel hooks stay reachable through the wrapper
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 61, (2, 2, 4, 8), generator=g)       # [micro-batch, rank, batch, tokens]
    loss_of = lambda m, x: m(x)["logits"].float().logsumexp(-1).mean()  # noqa: E731
    # single process: mean over both ranks' samples, two micro-batches accumulated
    for mb in range(2):
        (loss_of(ref, data[mb].reshape(8, 8)) / 2).backward()
    # two ranks: each sees its own half; gradients are averaged across ranks on the last micro-batch only
    for mb in range(2):
        with accumulation_context(ddp, is_last_microbatch=(mb == 1)):
            (loss_of(ddp, data[mb, rank]) / 2).backward()
    worst = 0.0
    for (n, p), q in zip(ref.named_parameters(), ddp.module.parameters()):
        worst = max(worst, (p.grad - q.grad).abs().max().item())
    assert worst < 1e-6, worst
    coll.barrier()
    print("DDP_OK", rank, worst)
    coll.close()


if __name__ == "__main__":
    main()
