"""Decode attention, fused sampler and cached generation on the GPU against PyTorch fp32 statements."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hd,Hq,Hk,window,splits", [(128, 8, 2, None, 1), (128, 16, 8, None, 4), (64, 12, 12, None, 1),
                                                     (128, 40, 8, None, 2), (128, 8, 4, 48, 1), (64, 8, 2, 100, 3)])
def test_decode_attention_matches_reference(hd, Hq, Hk, window, splits):
    from optimus_dl_b200.ops import decode as dec_ops

    torch.manual_seed(0)
    dev = torch.device("cuda")
    B, Tmax = 5, 333
    lens = torch.tensor([1, 64, 65, 200, 333], dtype=torch.int32, device=dev)
    kc = torch.randn(B, Tmax, Hk, hd, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(B, Tmax, Hk, hd, device=dev, dtype=torch.bfloat16)
    qkv = torch.randn(B, (Hq + 2 * Hk) * hd, device=dev, dtype=torch.bfloat16)
    q = qkv[:, : Hq * hd].unflatten(1, (Hq, hd))
    kn = qkv[:, Hq * hd:(Hq + Hk) * hd].unflatten(1, (Hk, hd))
    vn = qkv[:, (Hq + Hk) * hd:].unflatten(1, (Hk, hd))
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ref = dec_ops.decode_attention_ref(q.float(), kn.float(), vn.float(), kc_ref, vc_ref, lens, window=window)
    out = dec_ops.decode_attention(q, kn, vn, kc, vc, lens, window=window, n_splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref), "cache append differs"
    err = (out.float() - ref.float()).abs().max().item()
    assert err < 2e-2, err


def test_sampler_greedy_and_support():
    from optimus_dl_b200.ops import decode as dec_ops

    torch.manual_seed(0)
    dev = torch.device("cuda")
    B, V = 16, 50257
    logits = torch.randn(B, V, device=dev) * 3
    assert torch.equal(dec_ops.sample(logits, greedy=True), logits.argmax(-1))
    assert torch.equal(dec_ops.sample(logits.bfloat16(), greedy=True), logits.bfloat16().float().argmax(-1))
    for kw in (dict(top_k=50), dict(top_p=0.9), dict(top_k=200, top_p=0.5), dict(temperature=0.7, top_p=0.95)):
        allowed = torch.isfinite(dec_ops.filter_logits(logits, kw.get("temperature", 1.0), kw.get("top_k"), kw.get("top_p")))
        seen = torch.zeros_like(allowed)
        for step in range(64):
            s = dec_ops.sample(logits, seed=7, offset=step, **kw)
            assert allowed[torch.arange(B, device=dev), s].all(), kw
            seen[torch.arange(B, device=dev), s] = True
        assert seen.sum(-1).min() > 3, "sampler does not explore the kept set"


def test_sampler_distribution():
    from optimus_dl_b200.ops import decode as dec_ops

    dev = torch.device("cuda")
    z = torch.tensor([0.0, 1.0, 2.0, -5.0, 0.5], device=dev).repeat(8192, 1)
    s = dec_ops.sample(z, temperature=1.0, seed=3, offset=0)
    freq = torch.bincount(s, minlength=5).float() / s.numel()
    assert torch.allclose(freq, torch.softmax(z[0], -1), atol=0.02), freq
    s2 = dec_ops.sample(z, temperature=1.0, seed=3, offset=1)
    assert not torch.equal(s, s2)
    assert torch.equal(s, dec_ops.sample(z, temperature=1.0, seed=3, offset=0)), "same seed and offset must repeat"


@pytest.mark.parametrize("kind", ["llama", "qwen3", "gpt2"])
def test_cached_decode_logits_match_full_forward(kind):
    from optimus_dl_b200.models.gpt2 import GPT, GPTConfig
    from optimus_dl_b200.models.llama2 import Llama, LlamaConfig
    from optimus_dl_b200.models.qwen3 import Qwen3, Qwen3Config
    from optimus_dl_b200.recipe.generation import DecodeSession, generate

    torch.manual_seed(0)
    dev = torch.device("cuda")
    base = dict(n_layer=2, n_head=4, n_embd=256, vocab_size=512)
    if kind == "llama":
        model = Llama(LlamaConfig(n_kv_head=2, sequence_length=256, intermediate_size=512, **base))
    elif kind == "qwen3":
        model = Qwen3(Qwen3Config(n_kv_head=2, head_dim=64, sequence_length=256, intermediate_size=512, **base))
    else:
        model = GPT(GPTConfig(block_size=256, **base))
    model = model.to(device=dev, dtype=torch.bfloat16).eval()
    B, T0, n_new = 3, 70, 5
    ids = torch.randint(0, 512, (B, T0 + n_new), device=dev)
    with torch.no_grad():
        full = model(ids)["logits"].float()
        with DecodeSession(model, B, T0 + n_new) as sess:
            lg = sess.prefill(ids[:, :T0]).float()
            assert (lg - full[:, T0 - 1]).abs().max().item() < 0.1
            for i in range(n_new - 1):
                for use_graph in ((True,) if i else (False,)):
                    lg = sess.step(ids[:, T0 + i], use_graph=use_graph).float()
                err = (lg - full[:, T0 + i]).abs().max().item()
                assert err < 0.12, (i, err)
    out = generate(model, ids[:, :T0], 8, greedy=True)
    assert out.shape == (B, 8)
