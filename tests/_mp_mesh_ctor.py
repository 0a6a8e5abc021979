"""Worker: ``MeshCollective`` built directly with the reference's constructor arguments on two Gloo ranks
(optimus_dl/modules/distributed/mesh.py:66-77). Run under torchrun-style environment variables."""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def main() -> None:
    from optimus_dl_b200.parallel.collective import MeshCollective

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    coll = MeshCollective(rank=rank, world_size=world, local_world_size=world, local_rank=rank, device_type="cpu",
                          tp_size=world)
    assert coll.rank == rank and coll.world_size == 2 and coll.tp_world_size == 2 and coll.dp_world_size == 1
    assert coll.local_rank == rank and coll.tp_mesh is not None
    t = torch.tensor([float(rank + 1)])
    coll.tp_world.all_reduce(t)
    assert t.item() == 3.0
    # positional form, same order; an absent sharding size means "the ranks of this node divided by tp_size"
    again = MeshCollective(rank, world, world, rank, "cpu", None, None, 1)
    assert again.tp_world_size == 1 and again.dp_world_size == 2 and again.shard_world_size == 2
    print("MESH_CTOR_OK", flush=True)


if __name__ == "__main__":
    main()
