"""Every shipped root config composes, resolves and validates against its recipe's config schema."""

import os

import pytest

from optimus_dl_b200.core import compose, conf
from optimus_dl_b200.core.config_utils import non_resolving_instantiate

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")


@pytest.mark.parametrize("name", ["train_llama", "train_llama_efficient", "train_llama_fp8", "train_llama_pretokenized",
                                  "train_llama_shakespeare", "train_gpt2_speedrun", "train_synthetic"])
def test_train_configs_compose(name):
    cfg = compose.compose([os.path.join(ROOT, "train")], name, [])
    cfg = non_resolving_instantiate(cfg)
    # fields that only exist as defaults of the recipe's structured config (filled in when the recipe is built)
    for key, default in (("exp_tags", []), ("exp_description", None)):
        if key not in cfg.common:
            cfg.common[key] = default
    plain = conf.to_container(cfg, resolve=True)
    assert plain["_name"] == "base"
    assert plain["optimization"]["iterations"] > 0
    assert isinstance(plain["model_transforms"], list)
    if name == "train_llama_efficient":
        assert plain["model"]["_name"] == "llama2-7b" and plain["optimization"]["acc_steps"] == 32
        assert plain["data"]["scratch"]["base_transforms"]["transforms"][1]["max_seq_len"] == 4096
    if name == "train_gpt2_speedrun":
        assert plain["optimization"]["optimizer"]["_name"] == "muon"
        assert plain["criterion"]["softcap_type"] == "sigmoid"
    if name == "train_llama_fp8":
        assert plain["optimization"]["amp"]["fp8"]["enabled"] is True
        assert plain["model_transforms"][0]["_name"] == "transformer_engine"


@pytest.mark.parametrize("group,name,overrides", [
    ("eval", "quick", ["common.checkpoint_path=null"]), ("metrics", "default", []), ("serve", "char_shakespeare", []),
    ("serve", "tinyllama", []), ("prepare_data", "default", []), ("grpo", "default", []),
    ("eval", "quick_pretrained", []), ("metrics", "tinystories_test", [])])
def test_other_configs_compose(group, name, overrides):
    cfg = compose.compose([os.path.join(ROOT, group)], name, overrides)
    assert conf.is_config(cfg)
    if group == "prepare_data":
        assert cfg.tokenizer._name == "tiktoken" and cfg.processing.dtype == "uint16"
    if group == "grpo":
        assert conf.to_container(cfg, resolve=True)["grpo"]["group_size"] == 8
    if name == "quick_pretrained":                      # inherits the task list of ``quick`` and names a hub model
        plain = conf.to_container(cfg, resolve=True)
        assert plain["lm_eval"]["tasks"] == ["hellaswag", "arc_easy"] and plain["common"]["checkpoint_path"] is None
        assert plain["common"]["tokenizer"]["name"] == plain["common"]["model"]["hf_model_name"]
    if name == "tinystories_test":
        plain = conf.to_container(cfg, resolve=True)
        assert [m["_name"] for m in plain["metrics"]["tinystories"]] == ["accuracy", "perplexity", "loss"]
        assert plain["data"]["eval_datasets"]["tinystories"]["transform"]["transforms"][2]["batch_size"] == 4
        assert plain["loggers"][0]["output_dir"].startswith(plain["common"]["output_path"])


def test_transformer_engine_variants_parse():
    cfg = conf.load(os.path.join(ROOT, "model", "transforms", "transformer_engine.yaml"))
    assert set(cfg.keys()) >= {"_default", "full", "linear_only", "norm_only", "disabled"}
    from optimus_dl_b200.model_transforms import build_model_transform

    for key in cfg.keys():
        assert build_model_transform(cfg[key]) is not None


@pytest.mark.parametrize("preset,recipe", [("fp8_delayed", "delayed"), ("fp8_tensorwise", "tensorwise"),
                                           ("fp8_blockwise", "blockwise"), ("fp8_hybrid", None), ("fp8_e4m3", None)])
def test_fp8_amp_presets_compose(preset, recipe):
    cfg = compose.compose([os.path.join(ROOT, "train")], "train_llama_fp8", [f"optimization/amp={preset}"], apply_env=False)
    fp8 = cfg["optimization"]["amp"]["fp8"]
    assert fp8["enabled"] and fp8.get("recipe") == recipe        # None: the default recipe of Fp8Config (delayed) applies


@pytest.mark.parametrize("name", sorted(f[:-5] for f in os.listdir(os.path.join(ROOT, "train"))
                                        if f.startswith("train_") and f.endswith(".yaml")))
def test_train_configs_build_their_components(name, monkeypatch):
    """Every train root config yields a buildable model (on the meta device), criterion, schedule, model transforms,
    data transform and metric engines: no key in the shipped YAML is unknown to the code."""
    import torch

    from optimus_dl_b200.core.config_utils import non_resolving_instantiate
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.data.transforms import build_transform
    from optimus_dl_b200.lr_scheduler import build_lr_scheduler
    from optimus_dl_b200.metrics.engine import MetricEngine
    from optimus_dl_b200.model_transforms import build_model_transform
    from optimus_dl_b200.models import build_model

    monkeypatch.setenv("SCRATCH_HOME", "/tmp/optimus-test")
    monkeypatch.setenv("PERSISTENT_PATH", "/tmp/optimus-test")
    cfg = non_resolving_instantiate(compose.compose([os.path.join(ROOT, "train")], name, [], apply_env=False))
    with torch.device("meta"):
        model = build_model(cfg.model)
    assert sum(p.numel() for p in model.parameters()) > 0
    build_criterion(cfg.criterion)
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    build_lr_scheduler(cfg.lr_scheduler, optimizer=opt, iterations=int(cfg.optimization.iterations))
    for t in (cfg.get("model_transforms") or []):
        build_model_transform(t)
    train = cfg.data.get("train_datasets", {})
    if train and train.get("transform") is not None:
        build_transform(train.transform, device=torch.device("cpu"))
    metrics = cfg.get("metrics")
    if metrics and hasattr(metrics, "items"):
        for group, configs in metrics.items():
            MetricEngine(group, configs)
