"""Checkpoint manager (optimus_dl/modules/checkpoint/checkpoint_manager.py:70-905).

Disk layout (unchanged from the reference)::

    {out}/checkpoint_{iter:09d}/                 DCP directory, keys "model.*" and "optimizer.*"
    {out}/metadata_{iter:09d}.pt                 iteration, config, world_size, lr_scheduler, extras
    {out}/per_rank_metadata_{rank}_{iter:09d}.pt iteration, data_loaders, metrics, other stateful objects
    {out}/checkpoint_latest, metadata_latest.pt, per_rank_metadata_{rank}_latest.pt
                                                 symlinks to the newest persistent files, or real files
                                                 when only a rolling "last" checkpoint is kept

Every file is first written under a ``.tmp`` name; after a barrier the temporaries are renamed, so
a crash in the middle of a save leaves the previous ``*_latest`` untouched. ``metadata_only`` rewrites
just the metadata (used after an evaluation finished). Model and optimizer go through
``torch.distributed.checkpoint`` as sharded DTensors (``parallel/state.py``), so world sizes may
change between save and load; per-rank files are keyed by rank.
"""

from __future__ import annotations

import logging
import os
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Any, NamedTuple

import torch

from ..core import conf
from ..core.registry import RegistryConfig
from ..metrics import base as meters
from ..parallel import state as pstate
from .load_strategy import LoadStrategy

logger = logging.getLogger(__name__)


@dataclass
class CheckpointManagerConfig(RegistryConfig):
    pass


class CheckpointPath(NamedTuple):
    """``metadata`` file and ``checkpoint`` (weights) path of one save."""

    metadata: str
    checkpoint: str

    def per_rank_metadata(self, rank: int) -> str:
        """Path of ``rank``'s per-rank metadata file that belongs to this save."""
        p = Path(self.metadata)
        return str(p.with_name(p.name.replace("metadata_", f"per_rank_metadata_{rank}_", 1)))

    def is_dcp_checkpoint(self) -> bool:
        """A directory holds a sharded (``torch.distributed.checkpoint``) save; a file is a plain ``torch.save``."""
        return Path(self.checkpoint).is_dir()


def dcp_save(state_dict: dict, path: str, process_group: Any = None) -> None:
    import torch.distributed.checkpoint as dcp

    dcp.save(state_dict, storage_writer=dcp.FileSystemWriter(path), process_group=process_group)


def dcp_load(state_dict: dict, path: str, process_group: Any = None) -> None:
    import torch.distributed.checkpoint as dcp

    dcp.load(state_dict, storage_reader=dcp.FileSystemReader(path), process_group=process_group)


class _FakeColl:
    rank, world_size, is_master, tp_world_size, tp_rank = 0, 1, True, 1, 0
    process_group = None

    def barrier(self):
        pass

    def broadcast_objects(self, objs, src=0):
        pass


class CheckpointManager:
    def __init__(self, cfg: Any = None, output_path: str | None = None, checkpoint_path: str | os.PathLike | None = None,
                 save_freq: int | None = None, last_save_freq: int | None = None, **kwargs: Any):
        """``checkpoint_path`` is the reference's name for ``output_path``; ``save_freq`` / ``last_save_freq`` given
        here are the defaults of ``save_checkpoint_if_needed``."""
        self.cfg = cfg
        output_path = output_path if output_path is not None else checkpoint_path
        self.output_path = Path(output_path) if output_path is not None else None
        self.save_freq, self.last_save_freq = save_freq, last_save_freq

    # ------------------------------------------------------------------ discovery
    def is_restart(self, checkpoint_path: str | os.PathLike | None = None) -> bool:
        root = Path(checkpoint_path) if checkpoint_path is not None else self.output_path
        return root is not None and (root / "metadata_latest.pt").exists()

    def get_checkpoint(self, path: str | os.PathLike) -> CheckpointPath | None:
        """Accepts an output dir, a ``checkpoint_*`` dir, a ``metadata_*.pt`` file or ``metadata_latest.pt``."""
        p = Path(path)
        if p.is_dir() and p.name.startswith("checkpoint_"):
            suffix = p.name[len("checkpoint_"):]
            meta = p.parent / f"metadata_{suffix}.pt"
            return CheckpointPath(str(meta), str(p)) if meta.exists() else None
        if p.is_file() and p.name.startswith("metadata_"):
            suffix = p.name[len("metadata_"):-len(".pt")]
            return CheckpointPath(str(p), str(p.parent / f"checkpoint_{suffix}"))
        if p.is_dir():
            meta = p / "metadata_latest.pt"
            if meta.exists():
                return CheckpointPath(str(meta), str(p / "checkpoint_latest"))
        return None

    # ------------------------------------------------------------------ save
    def save_checkpoint_if_needed(self, iteration: int, *positional: Any, save_freq: int | None = None,
                                  last_save_freq: int | None = None, force_save: bool = False, **kwargs: Any) -> bool:
        """``(iteration, save_freq, last_save_freq, force_save, **save_kwargs)`` or, as the reference calls it,
        ``(iteration, collective, checkpoint_path, save_freq=..., last_save_freq=..., force_save=..., **save_kwargs)``.
        A numbered (persistent) checkpoint every ``save_freq`` iterations, a ``*_latest`` one every ``last_save_freq``."""
        if positional and (positional[0] is None or isinstance(positional[0], (int, bool))):
            names = ("save_freq", "last_save_freq", "force_save")
            given = dict(zip(names, positional))
            save_freq = given.get("save_freq", save_freq)
            last_save_freq = given.get("last_save_freq", last_save_freq)
            force_save = given.get("force_save", force_save)
        elif positional:
            kwargs.update(zip(("collective", "checkpoint_path"), positional))
        save_freq = self.save_freq if save_freq is None else save_freq
        last_save_freq = self.last_save_freq if last_save_freq is None else last_save_freq
        persistent = bool(save_freq) and save_freq > 0 and iteration % save_freq == 0
        last = bool(last_save_freq) and last_save_freq > 0 and iteration % last_save_freq == 0
        if last_save_freq is None or not last_save_freq:
            last = persistent       # without a separate cadence the rolling checkpoint follows the numbered one
        # a forced save is always a numbered one (optimus_dl/modules/checkpoint/checkpoint_manager.py: force_save
        # makes the save persistent), with the *_latest names pointing at it
        persistent = persistent or bool(force_save)
        if not (persistent or last):
            return False
        self.save_checkpoint(iteration=iteration, is_save_persistent=persistent, is_save_last=last or persistent, **kwargs)
        return True

    def _names(self, iteration: int, rank: int, persistent: bool) -> dict[str, Path]:
        tag = f"{iteration:09d}" if persistent else "latest"
        out = self.output_path
        return {"ckpt": out / f"checkpoint_{tag}", "meta": out / f"metadata_{tag}.pt",
                "rank": out / f"per_rank_metadata_{rank}_{tag}.pt"}

    def save_checkpoint(self, iteration: int = 0, model: Any = None, optimizer: Any = None,
                        lr_scheduler: Any = None, collective: Any = None, full_config: Any = None,
                        persistent: bool = True, metadata_only: bool = False, extra_metadata: dict | None = None,
                        data_loaders: dict | None = None, checkpoint_path: str | os.PathLike | None = None,
                        is_save_persistent: bool | None = None, is_save_last: bool | None = None, **stateful: Any) -> None:
        """Called with keywords. ``checkpoint_path`` overrides the manager's output path; ``is_save_persistent`` is
        the reference's name for ``persistent`` (a numbered checkpoint that ``*_latest`` links
        point at); without it the checkpoint is written under the ``*_latest`` names themselves."""
        if is_save_persistent is not None:
            persistent = bool(is_save_persistent)
        # a numbered checkpoint normally becomes the target of the *_latest links; ``is_save_last=False`` writes the
        # numbered files only, and asking for neither kind is a caller error
        link_latest = True if is_save_last is None else bool(is_save_last)
        if is_save_persistent is not None and is_save_last is not None and not persistent and not link_latest:
            raise ValueError("save_checkpoint: neither a persistent nor a latest checkpoint was requested")
        if checkpoint_path is not None:
            self.output_path = Path(checkpoint_path)
        assert self.output_path is not None, "checkpoint manager has no output path"
        coll = collective or _FakeColl()
        out = self.output_path
        if coll.is_master:
            out.mkdir(parents=True, exist_ok=True)
        coll.barrier()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        names = self._names(iteration, coll.rank, persistent)
        tmp = {k: Path(str(v) + f".{iteration}.tmp") for k, v in names.items()}
        # stale temporaries of an earlier crashed save
        for p in out.glob(f"*.{iteration}.tmp"):
            if coll.is_master or p.name.startswith(f"per_rank_metadata_{coll.rank}_"):
                shutil.rmtree(p, ignore_errors=True) if p.is_dir() else p.unlink(missing_ok=True)
        coll.barrier()
        mesh = _shard_mesh(coll)
        if not metadata_only and model is not None:
            sd: dict[str, Any] = {"model": pstate.model_state_dict(model, mesh)}
            if optimizer is not None:
                sd["optimizer"] = pstate.optimizer_state_dict(model, optimizer, mesh)
            dcp_save(sd, str(tmp["ckpt"]), process_group=None if coll.world_size == 1 else coll.process_group)
        metadata = {"iteration": iteration,
                    "config": conf.to_container(full_config, resolve=True) if conf.is_config(full_config) else full_config,
                    "world_size": coll.world_size,
                    "lr_scheduler": lr_scheduler.state_dict() if lr_scheduler is not None else None}
        metadata.update(extra_metadata or {})
        if coll.is_master:
            torch.save(metadata, tmp["meta"])
        if not metadata_only:
            per_rank = {"iteration": iteration,
                        "data_loaders": {k: (v.state_dict() if hasattr(v, "state_dict") else v) for k, v in (data_loaders or {}).items()},
                        "metrics": meters.state_dict()}
            for k, obj in stateful.items():
                if obj is not None and hasattr(obj, "state_dict"):
                    per_rank[k] = obj.state_dict()
            torch.save(per_rank, tmp["rank"])
        coll.barrier()
        # commit: replace finals
        if coll.is_master:
            if not metadata_only and tmp["ckpt"].exists():
                _remove(names["ckpt"])
                tmp["ckpt"].rename(names["ckpt"])
            _remove(names["meta"])
            tmp["meta"].rename(names["meta"])
        if not metadata_only and tmp["rank"].exists():
            _remove(names["rank"])
            tmp["rank"].rename(names["rank"])
        coll.barrier()
        if persistent and link_latest:
            if coll.is_master:
                _symlink(names["meta"].name, out / "metadata_latest.pt")
                if not metadata_only or not (out / "checkpoint_latest").exists():
                    _symlink(names["ckpt"].name, out / "checkpoint_latest")
            if not metadata_only or not (out / f"per_rank_metadata_{coll.rank}_latest.pt").exists():
                _symlink(names["rank"].name, out / f"per_rank_metadata_{coll.rank}_latest.pt")
        coll.barrier()
        logger.info("saved %s checkpoint at iteration %d to %s", "metadata-only" if metadata_only else "full", iteration, out)

    # ------------------------------------------------------------------ load
    def load_checkpoint_if_exists(self, checkpoint_path: str | os.PathLike | None = None, **kwargs: Any) -> tuple[int, dict | None]:
        """Resume from ``checkpoint_path`` (default: the manager's output path) when it holds a checkpoint; returns
        ``(start_iteration, metadata)``."""
        root = Path(checkpoint_path) if checkpoint_path is not None else self.output_path
        if not self.is_restart(root):
            return 1, None
        metadata = self.load_checkpoint(str(root), **kwargs)
        return int(metadata["iteration"]) + 1, metadata

    def load_checkpoint(self, path: str | os.PathLike | None = None, model: torch.nn.Module | None = None, optimizer: Any = None,
                        lr_scheduler: Any = None, collective: Any = None, strategy: LoadStrategy | None = None,
                        data_loaders: dict | None = None, checkpoint_path: str | os.PathLike | None = None,
                        load_strategy: LoadStrategy | None = None, **stateful: Any) -> dict:
        """``checkpoint_path`` / ``load_strategy`` are the reference's names for ``path`` / ``strategy``."""
        path = path if path is not None else checkpoint_path
        strategy = strategy if strategy is not None else load_strategy
        assert path is not None, "load_checkpoint needs a path"
        coll = collective or _FakeColl()
        strategy = LoadStrategy.from_cfg(strategy)
        cp = self.get_checkpoint(path)
        if cp is None:
            raise FileNotFoundError(f"no checkpoint found at {path}")
        mesh = _shard_mesh(coll)
        want_model = strategy.load_model and model is not None
        want_opt = strategy.load_optimizer and optimizer is not None and model is not None
        if want_model or want_opt:
            sd: dict[str, Any] = {}
            if want_model:
                msd = pstate.model_state_dict(model, mesh)
                for k in list(msd):
                    if any(ig in k for ig in strategy.extra_ignore_keys):
                        msd.pop(k)
                sd["model"] = msd
            if want_opt:
                sd["optimizer"] = pstate.optimizer_state_dict(model, optimizer, mesh)
            dcp_load(sd, cp.checkpoint, process_group=None if coll.world_size == 1 else coll.process_group)
            if want_model:
                if pstate.engine_of(model) is None:
                    model.load_state_dict(sd["model"], strict=not strategy.extra_ignore_keys)
                else:
                    pstate.after_model_load(model)
            if want_opt:
                pstate.load_optimizer_state_dict(model, optimizer, sd["optimizer"])
        box = [torch.load(cp.metadata, map_location="cpu", weights_only=False) if coll.is_master else None]
        coll.broadcast_objects(box, src=0)
        metadata = box[0]
        if strategy.load_scheduler and lr_scheduler is not None and metadata.get("lr_scheduler") is not None:
            lr_scheduler.load_state_dict(metadata["lr_scheduler"])
        suffix = Path(cp.metadata).name[len("metadata_"):]
        rank_file = Path(cp.metadata).parent / f"per_rank_metadata_{coll.rank}_{suffix}"
        per_rank = torch.load(rank_file, map_location="cpu", weights_only=False) if rank_file.exists() else {}
        if per_rank and per_rank.get("iteration") != metadata.get("iteration"):
            raise RuntimeError(f"checkpoint corrupted: per-rank metadata of rank {coll.rank} is from iteration "
                               f"{per_rank.get('iteration')}, the checkpoint from {metadata.get('iteration')}")
        # tensor-parallel peers must read identical data: take the state of the group's first rank
        if strategy.load_dataloaders and data_loaders:
            states = per_rank.get("data_loaders", {})
            tp = getattr(coll, "tp_world", None)
            if tp is not None and getattr(coll, "tp_world_size", 1) > 1:
                b = [states]
                tp.broadcast_objects(b, src=0)
                states = b[0]
            for k, dl in data_loaders.items():
                if k in states and states[k] is not None and hasattr(dl, "load_state_dict"):
                    dl.load_state_dict(states[k])
        if strategy.load_metrics and per_rank.get("metrics"):
            meters.load_state_dict(per_rank["metrics"])
        for k, obj in stateful.items():
            if obj is None or k not in per_rank or not hasattr(obj, "load_state_dict"):
                continue
            if k == "data_sources" and not strategy.load_data_sources:
                continue
            obj.load_state_dict(per_rank[k])
        if not strategy.load_iteration:
            metadata = dict(metadata, iteration=0)
        return metadata

    # ------------------------------------------------------------------ model-only helpers
    def build_model_from_checkpoint(self, path: str | os.PathLike | None = None, device: Any = "cpu",
                                    checkpoint_path: str | os.PathLike | None = None, **build_kwargs: Any):
        """Rebuild the model from the config stored in the checkpoint's metadata and load its weights."""
        path = str(path if path is not None else checkpoint_path)
        from ..models import build_model

        cp = self.get_checkpoint(path)
        if cp is None:
            raise FileNotFoundError(f"no checkpoint found at {path}")
        metadata = torch.load(cp.metadata, map_location="cpu", weights_only=False)
        model = build_model(metadata["config"]["model"], **build_kwargs)
        self.load_model_state_dict(model, cp.checkpoint)
        return model.to(device), metadata

    def load_model_state_dict(self, model: torch.nn.Module, path: str | os.PathLike | None = None, strict: bool = True,
                              checkpoint_path: str | os.PathLike | None = None) -> None:
        """Load weights from a DCP directory (converted through a temporary torch.save file) or a ``.pt`` file."""
        path = str(path if path is not None else checkpoint_path)
        p = Path(path)
        if p.is_dir():
            import tempfile

            from torch.distributed.checkpoint.format_utils import dcp_to_torch_save

            with tempfile.TemporaryDirectory() as d:
                f = os.path.join(d, "full.pt")
                dcp_to_torch_save(str(p), f)
                full = torch.load(f, map_location="cpu", weights_only=False)
            sd = full.get("model", full)
        else:
            full = torch.load(p, map_location="cpu", weights_only=False)
            sd = full.get("model", full)
        sd = {k: v for k, v in sd.items() if isinstance(v, torch.Tensor)}
        target = model.state_dict()
        sd = {k: v.to(target[k].dtype) if k in target else v for k, v in sd.items()}
        model.load_state_dict(sd, strict=strict)


def _shard_mesh(coll: Any) -> Any:
    mesh = getattr(coll, "parallel_mesh", None)
    if mesh is None or coll.world_size == 1:
        return None
    return mesh["dp_shard"]


def _remove(p: Path) -> None:
    if p.is_symlink() or p.is_file():
        p.unlink()
    elif p.is_dir():
        shutil.rmtree(p)


def _symlink(target_name: str, link: Path) -> None:
    if link.is_dir() and not link.is_symlink():
        shutil.rmtree(link)   # a rolling "latest" directory from an earlier non-persistent save
    tmp = link.with_name(link.name + ".lnk")
    if tmp.is_symlink() or tmp.exists():
        tmp.unlink()
    os.symlink(target_name, tmp)
    os.replace(tmp, link)
