"""Spellings, signatures and error classes that code written against the reference relies on: each case below
was first met by running the reference's own tests against this package."""

import importlib
import sys
from unittest.mock import MagicMock, patch

import numpy as np
import pytest
import torch

from optimus_dl_b200.core import conf


def test_import_paths_of_the_reference_resolve_to_the_same_modules():
    import optimus_dl_b200.models.blocks.attention as real

    alias = importlib.import_module("optimus_dl_b200.model.blocks.attention")
    assert alias is real and alias.FLASH_ATTENTION_AVAILABLE is True and alias.FLEX_ATTENTION_AVAILABLE is True
    dist = importlib.import_module("optimus_dl_b200.distributed")
    from optimus_dl_b200.parallel import collective

    assert dist.MeshCollective is collective.MeshCollective and dist.FakeCollective is collective.FakeCollective
    utils = importlib.import_module("optimus_dl_b200.core.omegaconf_utils")
    assert callable(utils.non_resolving_instantiate)
    with patch("optimus_dl_b200.model.blocks.attention.FLEX_ATTENTION_AVAILABLE", False):
        assert real.FLEX_ATTENTION_AVAILABLE is False            # the alias and the module are one object
    assert real.FLEX_ATTENTION_AVAILABLE is True


def test_module_level_names_can_be_substituted_and_stay_lazy():
    import optimus_dl_b200.data.datasets.huggingface as hf
    import optimus_dl_b200.data.transforms.tokenize as tok
    import optimus_dl_b200.loggers.mlflow as ml
    import optimus_dl_b200.models.presets.hf_llama as preset
    import optimus_dl_b200.recipe.pretokenize.source as source

    assert callable(tok.build_tokenizer) and isinstance(ml.MLFLOW_AVAILABLE, bool)
    assert "load_dataset" not in vars(hf)                        # `datasets` is imported on first use only
    with patch("optimus_dl_b200.data.datasets.huggingface.load_dataset") as fake:
        fake.return_value = [{"text": "a"}, {"text": "b"}]
        ds = hf.HuggingFaceDataset(conf.create({"_name": "huggingface_dataset", "dataset_load_kwargs": {"path": "x"}}))
        ds.reset()
        assert fake.call_args.kwargs["path"] == "x" and fake.call_args.kwargs["streaming"] is True
    assert hasattr(source, "list_repo_files") and hasattr(source, "hf_hub_download")
    hf_cfg = MagicMock()
    hf_cfg.num_hidden_layers, hf_cfg.num_attention_heads, hf_cfg.num_key_value_heads = 2, 4, 2
    hf_cfg.hidden_size, hf_cfg.intermediate_size, hf_cfg.vocab_size = 32, None, 100
    hf_cfg.max_position_embeddings, hf_cfg.rms_norm_eps, hf_cfg.rope_theta = 64, 1e-5, 10000.0
    hf_cfg.tie_word_embeddings, hf_cfg.rope_scaling, hf_cfg.head_dim = False, None, None
    hf_cfg.attention_bias = False
    from optimus_dl_b200.models import build_model

    with patch("optimus_dl_b200.models.presets.hf_llama.AutoConfig") as auto:
        auto.from_pretrained.return_value = hf_cfg
        model = build_model({"_name": "preset_hfllama2", "hf_model_name": "mock", "load_weights": False})
        auto.from_pretrained.assert_called_once_with("mock")
    assert model.config.n_layer == 2 and model.config.n_kv_head == 2 and model.head_dim == 8
    assert "AutoConfig" not in vars(preset)


def test_error_classes_match_every_except_clause_the_reference_allows():
    from optimus_dl_b200.core.registry import ConfigValidationError
    from optimus_dl_b200.ops.attention import BoundaryError, build_doc_start

    assert issubclass(ConfigValidationError, (ValueError,)) and issubclass(ConfigValidationError, TypeError)
    assert issubclass(ConfigValidationError, AssertionError)
    with pytest.raises(AssertionError, match="start with 0"):
        build_doc_start(1, 16, torch.device("cpu"), cu_seqlens=torch.tensor([1, 5, 16]))
    with pytest.raises(ValueError, match="match sequence length T"):
        build_doc_start(1, 16, torch.device("cpu"), cu_seqlens=torch.tensor([0, 5, 9]))
    assert issubclass(BoundaryError, ValueError)
    from optimus_dl_b200.core.config_utils import non_resolving_instantiate

    loop = non_resolving_instantiate(conf.create({"a": {"_target_": "builtins.dict", "ref": "${b}"},
                                                   "b": {"_target_": "builtins.dict", "ref": "${a}"}}))
    with pytest.raises(ValueError, match="Circular dependency detected"):
        loop.a
    own = non_resolving_instantiate(conf.create({"a": {"b": {"_target_": "builtins.dict", "val": 10.5, "ref": "${a.b.val}"}}}))
    assert own.a.b.ref == 10.5 and own.a.b.val == 10.5          # an absolute path to the block's own parameter
    from optimus_dl_b200.core.dtype import str_to_dtype

    with pytest.raises(ValueError, match="Unsupported dtype string"):
        str_to_dtype("invalid_dtype")
    from optimus_dl_b200.amp import get_fp8_format_from_string, Fp8Format

    assert get_fp8_format_from_string("float8_e4m3fn") is Fp8Format.E4M3 and get_fp8_format_from_string("fp8_hybrid") is Fp8Format.HYBRID
    assert get_fp8_format_from_string("e5m2fn") is Fp8Format.E5M2
    with pytest.raises(ValueError, match="Unknown FP8 format"):
        get_fp8_format_from_string("nope")


def test_sharder_inspection_properties_and_fractional_shard_size(tmp_path):
    from optimus_dl_b200.recipe.pretokenize.config import OutputConfig, ProcessingConfig
    from optimus_dl_b200.recipe.pretokenize.sharder import Sharder

    sh = Sharder(OutputConfig(dir=str(tmp_path), name="s"), ProcessingConfig(shard_size_mb=0.001))   # about 1 KB
    sh.dtype = np.uint16
    assert sh.add(list(range(400))) is False and sh.current_shard_size_bytes == 800
    assert sh.add(list(range(200))) is True and sh.shard_idx == 1          # 1200 bytes would not fit: flushed first
    assert len(np.load(tmp_path / "s_0000000000.npy")) == 400
    assert sh.current_shard_tokens == list(range(200)) and sh.current_shard_doc_lens == [200]
    other = Sharder(OutputConfig(dir=str(tmp_path), name="s"), ProcessingConfig(shard_size_mb=0.001))
    other.load_state(sh.get_state())
    assert other.current_shard_tokens == list(range(200)) and other.total_tokens == 400 and other.shard_idx == 1


def test_evaluator_takes_an_output_path_counts_batches_and_accepts_the_reference_argument_order(tmp_path):
    from optimus_dl_b200.checkpoint.eval_checkpoint_manager import EvaluationCheckpointManager
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.models import build_model
    from optimus_dl_b200.recipe.train.mixins.managers.evaluation_manager import Evaluator

    torch.manual_seed(0)
    model = build_model({"_name": "llama2", "n_layer": 1, "n_head": 2, "n_embd": 32, "vocab_size": 50, "sequence_length": 16,
                         "multiple_of": 8})
    crit = build_criterion({"_name": "cross_entropy"})

    class Loader:
        def __init__(self):
            self.pos = 0

        def __iter__(self):
            return self

        def __next__(self):
            if self.pos >= 4:
                raise StopIteration
            self.pos += 1
            g = torch.Generator().manual_seed(self.pos)
            return {"input_ids": torch.randint(0, 50, (2, 9), generator=g)}

        def state_dict(self):
            return {"pos": self.pos}

        def load_state_dict(self, s):
            self.pos = s["pos"]

    class Pipe:
        eval_freq = eval_iterations = eval_guaranteed_same_batches = eval_checkpointing = None

        def __init__(self):
            self.dataloader = Loader()

    ev = Evaluator(eval_freq=1, eval_checkpointing=2, output_path=str(tmp_path))
    assert isinstance(ev.eval_checkpoint_manager, EvaluationCheckpointManager) and ev.output_path == str(tmp_path)
    out = ev.run_evaluation(model=model, criterion=crit, eval_data_dict={"d": Pipe()}, device=torch.device("cpu"),
                            max_iterations=4, collective=None, all_metrics_configs={}, metrics_prefix="eval",
                            show_progress=False, iteration=7)
    assert out["eval/d"]["num_batches"] == 4
    saved = ev.eval_checkpoint_manager.read_iteration_state(7, "d")
    assert saved["eval_iterations_processed"] == 4 and saved["dataloader_state"] == {"pos": 4} and saved["rank"] == 0
    assert (tmp_path / "eval_checkpoints_iter_7" / "d_rank_0.pt").exists()
    # a second evaluator pointed at the same place resumes: nothing is left to do, the meters come from the file
    again = Evaluator(eval_freq=1, eval_checkpointing=2)
    again.eval_checkpoint_manager = EvaluationCheckpointManager(str(tmp_path))
    out2 = again.run_evaluation(model, crit, {"d": Pipe()}, torch.device("cpu"), 4, None, {}, "eval", False, 7)
    assert out2["eval/d"]["num_batches"] == 4 and out2["eval/d"]["loss"] == pytest.approx(out["eval/d"]["loss"])
    # without an iteration nothing is read or written
    free = Evaluator(eval_freq=1, output_path=str(tmp_path / "other"))
    assert free.run_evaluation(model, crit, {"d": Pipe()})["eval/d"]["num_batches"] == 4
    assert not (tmp_path / "other").exists()


def test_rmsnorm_helper_and_attention_dropout_modules():
    from optimus_dl_b200.models.blocks.attention import RotarySelfAttention
    from optimus_dl_b200.models.blocks.layer_norms import RMSNorm

    n = RMSNorm(16, eps=1e-6)
    x = torch.randn(3, 16)
    assert torch.allclose(n._norm(x) * n.weight, n(x), atol=1e-5)
    att = RotarySelfAttention(n_embd=32, n_head=4, dropout=0.25)
    assert isinstance(att.attn_dropout, torch.nn.Dropout) and att.attn_dropout.p == 0.25 and att.resid_dropout.p == 0.25


def test_mesh_collective_constructor_forms_on_two_gloo_ranks(unique_port):
    import os
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(unique_port), str(root / "tests" / "_mp_mesh_ctor.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0 and res.stdout.count("MESH_CTOR_OK") == 2, res.stdout[-2000:] + res.stderr[-3000:]
