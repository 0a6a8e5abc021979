"""Worker for the tensor-parallel correctness tests: compares a tensor-parallel model against the
same model run unsharded in this process. Run as ``python _mp_tp_check.py <backend> <model> <sp> <port>``
under torchrun-style environment variables (RANK, WORLD_SIZE)."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    backend, kind, sp, port = sys.argv[1], sys.argv[2], sys.argv[3] == "1", sys.argv[4]
    use_fp8 = len(sys.argv) > 5 and sys.argv[5] == "fp8"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = port
    cuda = backend == "nccl"
    if cuda:
        torch.cuda.set_device(rank)
    dist.init_process_group(backend, rank=rank, world_size=world)
    device = torch.device("cuda", rank) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32

    from optimus_dl_b200.criterion.cross_entropy import CrossEntropyCriterion, CrossEntropyCriterionConfig
    from optimus_dl_b200.models.llama2 import Llama, LlamaConfig
    from optimus_dl_b200.models.olmo3 import Olmo3, Olmo3Config
    from optimus_dl_b200.models.qwen3 import Qwen3, Qwen3Config

    torch.manual_seed(0)
    dims = dict(n_layer=2, n_head=4, n_kv_head=2, n_embd=256 if cuda else 64, vocab_size=512, sequence_length=256,
                tie_word_embeddings=False)
    if kind == "llama":
        cfg = LlamaConfig(intermediate_size=512 if cuda else 128, **dims)
        make = lambda: Llama(cfg)  # noqa: E731
    elif kind == "qwen3":
        cfg = Qwen3Config(intermediate_size=512 if cuda else 128, head_dim=64 if cuda else 16, **dims)
        make = lambda: Qwen3(cfg)  # noqa: E731
    else:
        cfg = Olmo3Config(intermediate_size=512 if cuda else 128, head_dim=64 if cuda else 16, sliding_window=64,
                          layer_types=["sliding_attention", "full_attention"], **dims)
        make = lambda: Olmo3(cfg)  # noqa: E731
    ref = make().to(device=device, dtype=dtype)
    par = make().to(device=device, dtype=dtype)
    par.load_state_dict(ref.state_dict())
    full_params = {n: p for n, p in ref.named_parameters()}
    par.apply_tp(dist.group.WORLD, sequence_parallel=sp, loss_parallel=True, device=device)

    B, T = 2, 128
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g).to(device)
    crit_ref = CrossEntropyCriterion(CrossEntropyCriterionConfig())
    crit_par = CrossEntropyCriterion(CrossEntropyCriterionConfig())
    loss_ref, _ = crit_ref(ref, {"input_ids": ids})
    loss_ref.backward()
    import contextlib

    fp8_ctx = contextlib.nullcontext()
    if use_fp8:
        from optimus_dl_b200.amp.fp8 import FP8Recipe
        from optimus_dl_b200.model_transforms.transformer_engine import mark_fp8_linears

        assert mark_fp8_linears(par) > 0
        fp8_ctx = FP8Recipe().autocast(True)
    with fp8_ctx:
        loss_par, _ = crit_par(par, {"input_ids": ids})
        loss_par.backward()
    if cuda:
        from optimus_dl_b200.ops import _lib

        torch.cuda.synchronize()
        _lib.check_status(device)
    tol = (6e-2 if use_fp8 else 3e-2) if cuda else 1e-4
    assert abs(loss_ref.item() - loss_par.item()) < tol, (loss_ref.item(), loss_par.item())
    # logits path (gathered over the vocabulary)
    with torch.no_grad():
        lr_ = ref(ids[:, :-1])["logits"].float()
        lp_ = par(ids[:, :-1])["logits"].float()
    assert lp_.shape == lr_.shape
    err = (lr_ - lp_).abs().max().item()
    assert err < (0.15 if cuda else 1e-3), f"logits differ by {err}"
    worst = 0.0
    for name, p in par.named_parameters():
        full = full_params[name].grad.float()
        dim = getattr(p, "_tp_shard_dim", None)
        if dim is not None:
            n = full.shape[dim] // world
            full = full.narrow(dim, rank * n, n)
        got = p.grad.float() if p.grad is not None else None
        assert got is not None, f"no gradient for {name}"
        scale = full.abs().max().item() + 1e-6
        e = (got - full).abs().max().item() / scale
        worst = max(worst, e)
        assert e < ((0.25 if use_fp8 else 6e-2) if cuda else 1e-3), f"gradient of {name} differs: rel {e}"
    if rank == 0:
        print(f"TP_OK kind={kind} sp={sp} loss={loss_par.item():.5f} worst_grad_rel={worst:.2e}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
