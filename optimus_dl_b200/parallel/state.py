"""Sharded state dicts of the FSDP engine, in the layout ``torch.distributed.checkpoint`` expects.

Model entries are the fp32 master shards and optimizer entries the fp32 moment shards, each
wrapped as a ``DTensor`` sharded on dim 0 over the shard group's mesh (plain tensors when the
world is one). Row ranges follow ``torch.chunk`` (the first ranks hold ``ceil(rows / world)`` rows),
which is also how FSDP2 shards, so checkpoints written here load under ``fully_shard`` in plain
PyTorch and the other way round. Tensors are views: loading in place updates the engine.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn


def _wrap(local: torch.Tensor, full_shape: tuple, mesh: Any) -> Any:
    if mesh is None:
        return local
    from torch.distributed.tensor import DTensor, Shard

    stride = torch.empty(full_shape, device="meta").stride()
    return DTensor.from_local(local, mesh, [Shard(0)], run_check=False, shape=torch.Size(full_shape), stride=stride)


def engine_of(model: nn.Module) -> Any:
    return getattr(model, "_sharding_engine", None)


def _tp_mesh_of(param: torch.Tensor) -> Any:
    tp = getattr(param, "_tp_state", None)
    if tp is None or tp.size == 1:
        return None
    if tp.mesh is None:
        from torch.distributed.device_mesh import DeviceMesh

        tp.mesh = DeviceMesh.from_group(tp.group, tp.device.type)
    return tp.mesh


def _wrap_tp(local: torch.Tensor, param: torch.Tensor) -> Any:
    """Tensor-parallel shard -> ``DTensor`` sharded on the parameter's tensor-parallel dimension, the layout
    ``parallelize_module`` gives the reference's parameters (row-sharded ``wq``, column-sharded ``wo``, ...)."""
    dim = getattr(param, "_tp_shard_dim", None)
    mesh = _tp_mesh_of(param)
    if dim is None or mesh is None:
        return local
    from torch.distributed.tensor import DTensor, Shard

    full = list(local.shape)
    full[dim] *= mesh.size(0)
    stride = torch.empty(full, device="meta").stride()
    return DTensor.from_local(local, mesh, [Shard(dim)], run_check=False, shape=torch.Size(full), stride=stride)


def _wrap_2d(local: torch.Tensor, inf_shape: tuple, param: torch.Tensor, dp_mesh: Any) -> Any:
    """Shard of a parameter that is split over tensor-parallel ranks first and over the data-parallel shard
    group second: a 2-D ``DTensor`` on ``(dp_shard, tp)``. When both splits hit dim 0 the data-parallel
    placement is the strided shard PyTorch uses for FSDP2 on top of tensor parallelism, so the global
    tensor keeps its natural row order."""
    from torch.distributed.device_mesh import DeviceMesh
    from torch.distributed.tensor import DTensor, Shard
    from torch.distributed.tensor.placement_types import _StridedShard

    tp_mesh = _tp_mesh_of(param)
    dim = int(param._tp_shard_dim)
    tp_size = tp_mesh.size(0)
    if dim == 0 and inf_shape[0] % dp_mesh.size(0) != 0:
        raise NotImplementedError("checkpointing uneven data-parallel shards of a row-split tensor-parallel parameter")
    root = getattr(tp_mesh, "_get_root_mesh", lambda: None)()
    mesh2d = root["dp_shard", "tp"] if root is not None and root is not tp_mesh and "dp_shard" in (root.mesh_dim_names or ()) \
        else None
    if mesh2d is None:
        raise NotImplementedError("tensor-parallel x sharded checkpoints need the (dp_shard, tp) device mesh")
    full = list(inf_shape)
    full[dim] *= tp_size
    dp_place = _StridedShard(0, split_factor=tp_size) if dim == 0 else Shard(0)
    stride = torch.empty(full, device="meta").stride()
    return DTensor.from_local(local, mesh2d, [dp_place, Shard(dim)], run_check=False, shape=torch.Size(full), stride=stride)


def _wrap_shard(local: torch.Tensor, inf: Any, use_mesh: Any) -> Any:
    """Checkpoint view of one engine shard: plain, 1-D (data-parallel or tensor-parallel) or 2-D ``DTensor``."""
    if len(inf.shape) == 0:
        return local
    tp_sharded = getattr(inf.param, "_tp_shard_dim", None) is not None and _tp_mesh_of(inf.param) is not None
    if tp_sharded and use_mesh is not None:
        return _wrap_2d(local, inf.shape, inf.param, use_mesh)
    if tp_sharded:
        return _wrap_tp(local.view(inf.shape), inf.param)
    return _wrap(local, inf.shape, use_mesh)


def model_state_dict(model: nn.Module, mesh: Any = None) -> dict[str, Any]:
    """``{fqn: tensor}``; engine-managed parameters appear as (sharded) fp32 master weights."""
    eng = engine_of(model)
    if eng is None:
        sd = dict(model.state_dict())
        if getattr(model, "_tp", None) is not None:
            params = dict(model.named_parameters(remove_duplicate=False))
            for name, p in params.items():
                if name in sd and getattr(p, "_tp_shard_dim", None) is not None:
                    sd[name] = _wrap_tp(sd[name], p)
        return sd
    out: dict[str, Any] = {}
    use_mesh = mesh if eng.world > 1 else None
    for name, g, inf in eng.named_sharded_state():
        out[name] = _wrap_shard(g.local_shard(inf, g.master), inf, use_mesh)
    # tied parameters appear once in named_parameters; mirror the aliases the module's own
    # state_dict would list (e.g. lm_head.weight == transformer.wte.weight)
    by_id = {id(p): n for n, p in model.named_parameters()}
    for n, p in model.named_parameters(remove_duplicate=False):
        if n not in out and id(p) in by_id and by_id[id(p)] in out:
            out[n] = out[by_id[id(p)]]
    for n, b in model.named_buffers():
        out[n] = b
    return out


def after_model_load(model: nn.Module) -> None:
    """Call after the master shards were overwritten: refresh bf16 rows and force a re-gather."""
    eng = engine_of(model)
    if eng is None:
        return
    for g in eng.groups:
        g.refresh_lp_from_master()
    if eng.world > 1:
        # every rank has rewritten its shard rows before any peer gathers them again
        eng.host_sync()
        if not any(g.pooled for g in eng.groups):
            eng.gather_all()
            eng.host_sync()


def optimizer_state_dict(model: nn.Module, optimizer: Any, mesh: Any = None) -> dict[str, Any]:
    """``{"state": {fqn: {step, exp_avg, exp_avg_sq}}, "param_groups": [...]}`` with sharded moments."""
    eng = engine_of(model)
    from .fsdp import ShardedAdamW

    if eng is None or not isinstance(optimizer, ShardedAdamW):
        # FQN-keyed and with the (possibly still empty) per-parameter state materialised, so that a
        # fresh optimizer can be filled in place by a checkpoint load
        from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict

        return _with_reference_group_keys(get_optimizer_state_dict(model, optimizer), adamw=False)
    use_mesh = mesh if eng.world > 1 else None
    state: dict[str, Any] = {}
    for name, g, inf in eng.named_sharded_state():
        g.ensure_state()
        state[name] = {
            "step": torch.tensor(float(optimizer.step_count)),
            "exp_avg": _wrap_shard(g.local_shard(inf, g.exp_avg), inf, use_mesh),
            "exp_avg_sq": _wrap_shard(g.local_shard(inf, g.exp_avg_sq), inf, use_mesh),
        }
    names = {id(p): n for n, p in model.named_parameters()}
    groups = []
    for pg in optimizer.param_groups:
        d = {k: v for k, v in pg.items() if k != "params"}
        d["params"] = [names[id(p)] for p in pg["params"]]
        groups.append(d)
    return _with_reference_group_keys({"state": state, "param_groups": groups}, adamw=True)


# what ``torch.optim.AdamW`` keeps in every parameter group; the reference's optimizer is that class, and a
# distributed-checkpoint load into it asks the checkpoint for each of these keys
_TORCH_ADAMW_GROUP_DEFAULTS = {"amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
                               "differentiable": False, "fused": True, "decoupled_weight_decay": True}


def _with_reference_group_keys(sd: dict[str, Any], adamw: bool) -> dict[str, Any]:
    """Parameter groups as the reference writes them: ``param_names`` beside ``params`` (torch records the names of
    parameters that were handed over as ``(name, parameter)`` pairs, which the reference does), and for this
    package's own AdamW the remaining keys of ``torch.optim.AdamW`` groups, so that either code base can load the
    other's optimizer state."""
    for g in sd.get("param_groups", []):
        g.setdefault("param_names", list(g.get("params", [])))
        if adamw:
            for k, v in _TORCH_ADAMW_GROUP_DEFAULTS.items():
                g.setdefault(k, v)
    return sd


def load_optimizer_state_dict(model: nn.Module, optimizer: Any, sd: dict[str, Any]) -> None:
    eng = engine_of(model)
    from .fsdp import ShardedAdamW

    if eng is None or not isinstance(optimizer, ShardedAdamW):
        from torch.distributed.checkpoint.state_dict import set_optimizer_state_dict

        set_optimizer_state_dict(model, optimizer, sd)
        return
    steps = [float(v["step"]) for v in sd.get("state", {}).values() if "step" in v]
    if steps:
        optimizer.step_count = int(max(steps))
    for pg, saved in zip(optimizer.param_groups, sd.get("param_groups", [])):
        # only what this optimizer keeps per group (a checkpoint also carries torch AdamW's other group keys)
        pg.update({k: v for k, v in saved.items() if k != "params" and k in pg})
