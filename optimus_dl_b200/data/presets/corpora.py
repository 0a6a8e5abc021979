"""Named corpora: ``preset_fineweb_edu``, ``preset_slimpajama6b``, ``preset_slimpajama``,
``preset_tinyshakespeare`` (optimus_dl/modules/data/presets/*.py)."""

from __future__ import annotations

from dataclasses import dataclass

from ...core import conf
from ...core.registry import RegistryConfigStrict
from ..datasets import register_dataset
from ..datasets.huggingface import HuggingFaceDataset
from ..datasets.txt_lines import TxtLinesDataset, TxtLinesDatasetConfig

TINY_SHAKESPEARE_URL = "https://raw.githubusercontent.com/karpathy/char-rnn/master/data/tinyshakespeare/input.txt"


@dataclass
class SplitConfig(RegistryConfigStrict):
    split: str = "train"
    streaming: bool = True


def _hf(load_kwargs: dict, rank: int, world_size: int) -> HuggingFaceDataset:
    return HuggingFaceDataset(conf.create({"dataset_load_kwargs": load_kwargs}), rank=rank, world_size=world_size)


@register_dataset("preset_slimpajama6b", SplitConfig)
def make_slimpajama_6b(cfg, rank: int = 0, world_size: int = 1, **_):
    return _hf({"path": "DKYoon/SlimPajama-6B", "split": cfg.split, "streaming": cfg.streaming}, rank, world_size)


@register_dataset("preset_slimpajama", SplitConfig)
def make_slimpajama(cfg, rank: int = 0, world_size: int = 1, **_):
    return _hf({"path": "cerebras/SlimPajama-627B", "split": cfg.split, "streaming": cfg.streaming}, rank, world_size)


@dataclass
class FinewebConfig(RegistryConfigStrict):
    subset: str = "sample-10BT"


@register_dataset("preset_fineweb_edu", FinewebConfig)
def make_fineweb_edu(cfg, rank: int = 0, world_size: int = 1, **_):
    return _hf({"path": "HuggingFaceFW/fineweb-edu", "split": "train", "name": cfg.subset}, rank, world_size)


@dataclass
class TinyShakespeareConfig(TxtLinesDatasetConfig):
    file_link: str = TINY_SHAKESPEARE_URL


@register_dataset("preset_tinyshakespeare", TinyShakespeareConfig)
def make_tinyshakespeare(cfg, rank: int = 0, world_size: int = 1, **_):
    return TxtLinesDataset(cfg, rank=rank, world_size=world_size)
