"""Worker: tensor-parallel model -> DCP checkpoint -> full tensors must equal the unsharded model's."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
import torch.distributed.checkpoint as dcp  # noqa: E402


def main() -> None:
    port, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = port
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from optimus_dl_b200.models.qwen3 import Qwen3, Qwen3Config
    from optimus_dl_b200.parallel.state import model_state_dict

    torch.manual_seed(0)
    cfg = Qwen3Config(n_layer=2, n_head=4, n_kv_head=2, head_dim=16, n_embd=64, vocab_size=128, sequence_length=64,
                      intermediate_size=128, tie_word_embeddings=False, attention_bias=True)
    ref = Qwen3(cfg)
    par = Qwen3(cfg)
    par.load_state_dict(ref.state_dict())
    par.apply_tp(dist.group.WORLD, sequence_parallel=True, device="cpu")
    sd = model_state_dict(par)
    from torch.distributed.tensor import DTensor

    n_dt = sum(isinstance(v, DTensor) for v in sd.values())
    assert n_dt >= 2 * 7 + 2, n_dt
    assert sd["transformer.h.0.attn.wq.weight"].shape == ref.transformer.h[0].attn.wq.weight.shape
    assert sd["transformer.h.0.attn.wo.weight"].placements[0].dim == 1
    dcp.save({"model": sd}, checkpoint_id=out_dir)
    dist.barrier()
    if rank == 0:
        from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

        f = os.path.join(out_dir, "full.pt")
        dcp_to_torch_save(out_dir, f)
        full = torch.load(f, map_location="cpu", weights_only=False)["model"]
        for name, t in ref.state_dict().items():
            assert name in full, name
            assert torch.equal(full[name], t), name
    dist.barrier()
    # load back into a differently initialised tensor-parallel model
    torch.manual_seed(123)
    other = Qwen3(cfg)
    other.apply_tp(dist.group.WORLD, sequence_parallel=True, device="cpu")
    sd2 = model_state_dict(other)
    dcp.load({"model": sd2}, checkpoint_id=out_dir)
    for (n1, p1), (n2, p2) in zip(par.named_parameters(), other.named_parameters()):
        assert torch.equal(p1, p2), n1
    if rank == 0:
        print("TP_CKPT_OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
