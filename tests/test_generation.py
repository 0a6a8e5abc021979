"""KV-cache generation against full-prefix recomputation, and the sampler's filtering rules (CPU)."""

import pytest
import torch

from optimus_dl_b200.models.gpt2 import GPT, GPTConfig
from optimus_dl_b200.models.llama2 import Llama, LlamaConfig
from optimus_dl_b200.models.olmo3 import Olmo3, Olmo3Config
from optimus_dl_b200.models.qwen3 import Qwen3, Qwen3Config
from optimus_dl_b200.ops import decode as dec_ops
from optimus_dl_b200.recipe.generation import generate, supports_kv_cache


def _models():
    torch.manual_seed(0)
    base = dict(n_layer=2, n_head=4, n_embd=64, vocab_size=97)
    yield "gpt2", GPT(GPTConfig(block_size=64, **base))
    yield "llama", Llama(LlamaConfig(n_kv_head=2, sequence_length=64, intermediate_size=128, **base))
    yield "qwen3", Qwen3(Qwen3Config(n_kv_head=2, head_dim=16, sequence_length=64, intermediate_size=128, **base))
    yield "olmo3", Olmo3(Olmo3Config(n_kv_head=2, head_dim=16, sequence_length=64, intermediate_size=128,
                                     sliding_window=8, layer_types=["sliding_attention", "full_attention"], **base))


@pytest.mark.parametrize("name,model", list(_models()))
def test_cached_generation_matches_recompute(name, model):
    assert supports_kv_cache(model)
    ids = torch.randint(0, 97, (3, 7), generator=torch.Generator().manual_seed(1))
    a = generate(model, ids, 12, greedy=True, use_kv_cache=True)
    b = generate(model, ids, 12, greedy=True, use_kv_cache=False)
    assert a.shape == (3, 12)
    assert torch.equal(a, b), name


def test_eos_stops_and_pads():
    _, model = next(_models())
    ids = torch.randint(0, 97, (2, 5), generator=torch.Generator().manual_seed(2))
    free = generate(model, ids, 6, greedy=True)
    eos = int(free[0, 1])
    out = generate(model, ids, 6, greedy=True, eos_token_id=eos)
    row = out[0].tolist()
    assert row[1] == eos and all(t == eos for t in row[2:])


def test_filter_rules():
    z = torch.tensor([[2.0, 1.0, 1.0, 0.0, -1.0]])
    k2 = dec_ops.filter_logits(z, 1.0, top_k=2)
    assert torch.isfinite(k2[0]).tolist() == [True, True, True, False, False]  # ties at the k-th value are kept
    p = torch.softmax(z, -1)[0]
    cut = float(p[0]) + 1e-4  # mass of the largest alone is below the threshold: the next ones are kept too
    kp = dec_ops.filter_logits(z, 1.0, top_p=cut)
    assert torch.isfinite(kp[0]).tolist()[0] and torch.isfinite(kp[0]).tolist()[1]
    assert not torch.isfinite(kp[0]).tolist()[4]
    first = dec_ops.filter_logits(z, 1.0, top_p=float(p[0]) - 1e-3)
    assert torch.isfinite(first[0]).tolist() == [True, False, False, False, False]


def test_sampling_follows_distribution():
    g = torch.Generator().manual_seed(0)
    z = torch.tensor([[0.0, 1.0, 2.0, -5.0]]).repeat(4000, 1)
    s = dec_ops.sample(z, temperature=1.0, generator=g)
    freq = torch.bincount(s, minlength=4).float() / s.numel()
    assert torch.allclose(freq, torch.softmax(z[0], -1), atol=0.03)
    assert torch.equal(dec_ops.sample(z[:4], greedy=True), torch.full((4,), 2))


def test_generation_source_drives_any_callable_that_returns_logits():
    """``GenerationSource`` (optimus_dl/modules/metrics/sources/generation.py:20-177) with a stand-in model: called once
    per new token with ``input_ids=``, greedy by default, per-sequence EOS with padding."""
    from optimus_dl_b200.metrics.source import StandardProtocols
    from optimus_dl_b200.metrics.sources.generation import GenerationSource, GenerationSourceConfig

    calls = {"n": 0}

    def successor(**kw):                                  # next token = last token + 1 (mod 20)
        calls["n"] += 1
        ids = kw["input_ids"]
        logits = torch.zeros(*ids.shape, 20)
        logits.scatter_(2, ((ids + 1) % 20)[..., None], 10.0)
        return {"logits": logits}

    out = GenerationSource(GenerationSourceConfig(max_new_tokens=5, do_sample=False))(
        dependencies={}, model=successor, batch={"input_ids": torch.tensor([[1, 2, 3]])})[StandardProtocols.GENERATED_TOKENS]
    assert torch.equal(out, torch.tensor([[4, 5, 6, 7, 8]])) and calls["n"] == 5
    out = GenerationSource(GenerationSourceConfig(max_new_tokens=10, do_sample=False, eos_token_id=7))(
        dependencies={}, model=successor, batch={"input_ids": torch.tensor([[1, 2, 3], [10, 11, 12]])})[StandardProtocols.GENERATED_TOKENS]
    assert out.shape == (2, 10) and out[0].tolist() == [4, 5, 6, 7] + [7] * 6 and out[1, 0].item() == 13
    noisy = lambda **kw: {"logits": torch.randn(1, kw["input_ids"].shape[1], 20)}  # noqa: E731
    out = GenerationSource(GenerationSourceConfig(max_new_tokens=2, do_sample=True, temperature=0.8, top_k=5, top_p=0.9))(
        dependencies={}, model=noisy, batch={"input_ids": torch.tensor([[1, 2, 3]])})[StandardProtocols.GENERATED_TOKENS]
    assert out.shape == (1, 2)
