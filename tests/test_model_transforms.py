"""Model transforms that need no process group: activation checkpointing, weight loading, the compile and
transformer_engine transforms (optimus_dl/modules/model_transforms/{checkpoint,load_weights,compile,
transformer_engine}.py) and the order in which the model builder applies them."""

import pytest
import torch

from optimus_dl_b200.checkpoint.checkpoint_manager import CheckpointManager
from optimus_dl_b200.model_transforms import build_model_transform
from optimus_dl_b200.models import build_model

CFG = dict(_name="llama2", n_layer=3, n_head=2, n_kv_head=1, n_embd=128, vocab_size=61, sequence_length=32, intermediate_size=256)


def _model(seed=0, **over):
    torch.manual_seed(seed)
    return build_model({**CFG, **over})


def _loss(m, x):
    return m(x)["logits"].float().logsumexp(-1).mean()


def test_activation_checkpoint_recomputes_and_changes_nothing_numerically():
    x = torch.randint(0, 61, (2, 16))
    plain, ckpt = _model(), _model()
    calls = {"n": 0}
    for blk in ckpt.transformer.h:
        orig = blk.forward

        def counted(*a, _o=orig, **k):
            calls["n"] += 1
            return _o(*a, **k)

        blk.forward = counted
    out = build_model_transform({"_name": "activation_checkpoint", "layer_classes": ["LlamaBlock", "RotaryTransformerBlock"]}).apply(ckpt)
    assert out is ckpt and set(ckpt.state_dict()) == set(plain.state_dict())      # parameter names are untouched
    from optimus_dl_b200.model_transforms.checkpoint import CheckpointWrapper
    blk0 = ckpt.transformer.h[0]
    assert isinstance(blk0, CheckpointWrapper) and blk0.module is blk0 and blk0.use_reentrant is False
    assert type(blk0).__name__ == type(plain.transformer.h[0]).__name__ and isinstance(blk0, type(plain.transformer.h[0]))
    _loss(plain, x).backward()
    _loss(ckpt, x).backward()
    assert calls["n"] == 2 * len(ckpt.transformer.h)                               # every block ran again in backward
    for (n, p), q in zip(plain.named_parameters(), ckpt.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6), n
    calls["n"] = 0
    with torch.no_grad():
        ckpt(x)
    assert calls["n"] == len(ckpt.transformer.h)                                   # no recomputation without gradients
    every_other = _model()
    build_model_transform({"_name": "activation_checkpoint", "layer_classes": ["LlamaBlock", "RotaryTransformerBlock"],
                           "every_nth": 2, "ops_to_save": ["torch.ops.aten.mm.default"]}).apply(every_other)
    _loss(every_other, x).backward()
    assert all(p.grad is not None for p in every_other.parameters())
    none = _model()
    build_model_transform({"_name": "activation_checkpoint", "layer_classes": ["NoSuchBlock"]}).apply(none)
    _loss(none, x).backward()


def test_load_weights_from_a_run_directory_a_file_and_skip_on_restart(tmp_path):
    src = _model(seed=1)
    CheckpointManager(output_path=str(tmp_path / "run")).save_checkpoint(iteration=7, model=src, full_config={"model": CFG})
    for path in (tmp_path / "run", tmp_path / "run" / "checkpoint_000000007", tmp_path / "run" / "metadata_latest.pt"):
        dst = _model(seed=2)
        build_model_transform({"_name": "load_weights", "checkpoint_path": str(path)}).apply(dst, is_restart=False)
        assert all(torch.equal(a, b) for a, b in zip(src.state_dict().values(), dst.state_dict().values())), path
    plain = tmp_path / "w.pt"
    torch.save(src.state_dict(), plain)
    dst = _model(seed=3)
    build_model_transform({"_name": "load_weights", "path": str(plain)}).apply(dst)
    assert torch.equal(dst.lm_head.weight, src.lm_head.weight)
    kept = _model(seed=4)
    before = kept.lm_head.weight.detach().clone()
    build_model_transform({"_name": "load_weights", "checkpoint_path": str(plain)}).apply(kept, is_restart=True)
    assert torch.equal(kept.lm_head.weight, before)                                # a restart keeps its own weights
    forced = _model(seed=4)
    build_model_transform({"_name": "load_weights", "checkpoint_path": str(plain), "skip_on_restart": False}).apply(forced, is_restart=True)
    assert torch.equal(forced.lm_head.weight, src.lm_head.weight)
    with pytest.raises(ValueError):
        build_model_transform({"_name": "load_weights"}).apply(_model())


def test_compile_transform_leaves_the_model_alone_unless_asked():
    m = _model()
    assert build_model_transform({"_name": "compile", "compile_kwargs": {"mode": "max-autotune"},
                                  "activation_memory_budget": 0.3}).apply(m) is m
    assert build_model_transform({"_name": "compile", "use_inductor": True, "compile_kwargs": {"disable": True}}).apply(m) is m


def test_transformer_engine_transform_marks_linears_and_pre_norms():
    m = _model()
    out = build_model_transform({"_name": "transformer_engine"}).apply(m)
    assert out is m
    marked = [n for n, p in m.named_parameters() if getattr(p, "_fp8", False)]
    assert len(marked) == 3 * 7 and all(".h." in n and n.endswith(".weight") for n in marked)   # q k v o + three MLP matrices
    assert not getattr(m.lm_head.weight, "_fp8", False)
    assert sum(bool(getattr(mod, "_fp8_out", False)) for mod in m.modules()) == 6               # ln_1, ln_2 of each block
    edge = _model()
    build_model_transform({"_name": "transformer_engine", "replace_norm": False,
                           "linear_kwargs": {"skip_first_layers": 1, "skip_last_layers": 1, "include_lm_head": True}}).apply(edge)
    marked = [n for n, p in edge.named_parameters() if getattr(p, "_fp8", False)]
    assert all(".h.1." in n or n.startswith(("lm_head", "transformer.wte")) for n in marked) and len(marked) == 7 + 1
    assert not any(getattr(mod, "_fp8_out", False) for mod in edge.modules())
    off = _model()
    build_model_transform({"_name": "transformer_engine", "enabled": False}).apply(off)
    build_model_transform({"_name": "transformer_engine", "replace_linear": False}).apply(off)
    assert not any(getattr(p, "_fp8", False) for p in off.parameters())
    narrow = _model(n_embd=96, intermediate_size=160)                                             # 96 is not a multiple of 128
    build_model_transform({"_name": "transformer_engine"}).apply(narrow)
    assert not any(getattr(p, "_fp8", False) for p in narrow.parameters())


def test_model_builder_applies_transforms_in_list_order(tmp_path):
    from optimus_dl_b200.recipe.mixins.model_builder import ModelBuilder

    src = _model(seed=9)
    torch.save(src.state_dict(), tmp_path / "w.pt")
    builder = ModelBuilder(model_transforms=[
        {"_name": "load_weights", "checkpoint_path": str(tmp_path / "w.pt")},
        {"_name": "transformer_engine"},
        {"_name": "activation_checkpoint", "layer_classes": ["LlamaBlock", "RotaryTransformerBlock"]},
        {"_name": "compile"},
    ])
    model = builder.build_model(CFG, device=torch.device("cpu"))
    assert torch.equal(model.lm_head.weight, src.lm_head.weight)
    assert any(getattr(p, "_fp8", False) for p in model.parameters())
    _loss(model, torch.randint(0, 61, (1, 8))).backward()


def test_compile_budget_turns_on_block_recomputation(caplog):
    """The reference's 7B recipe sets compile.activation_memory_budget: 0.3; without a compiler the budget is
    honoured by recomputing that share of the blocks, loudly."""
    import logging

    from optimus_dl_b200.model_transforms import build_model_transform
    from optimus_dl_b200.models import build_model

    model = build_model(dict(_name="llama2", n_layer=10, n_head=4, n_kv_head=2, n_embd=64, intermediate_size=128,
                             vocab_size=128, sequence_length=32, tie_word_embeddings=False))
    with caplog.at_level(logging.WARNING):
        out = build_model_transform({"_name": "compile", "activation_memory_budget": 0.3}).apply(model)
    assert out is model
    marked = [getattr(b, "_activation_checkpointed", False) for b in model.transformer.h]
    assert sum(marked) == 7
    assert any("recomputing 7 of 10" in r.message for r in caplog.records)
    import torch

    ids = torch.randint(0, 128, (2, 17))
    ref = build_model(dict(_name="llama2", n_layer=10, n_head=4, n_kv_head=2, n_embd=64, intermediate_size=128,
                           vocab_size=128, sequence_length=32, tie_word_embeddings=False))
    ref.load_state_dict(model.state_dict())
    la = model(input_ids=ids)["logits"].float().sum()
    lb = ref(input_ids=ids)["logits"].float().sum()
    la.backward()
    lb.backward()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-5), n
    again = build_model_transform({"_name": "compile", "activation_memory_budget": 1.0}).apply(ref)
    assert not any(getattr(b, "_activation_checkpointed", False) for b in again.transformer.h)
