"""Attention behaviours across model families on CPU: causality, batch independence, padding, sliding windows,
rotary position handling and gradient equivalence of packed batches (behaviours of
optimus_dl/modules/model/blocks/attention.py:44-536 and blocks/rope.py:13-253)."""

import math

import pytest
import torch

from optimus_dl_b200.models import build_model
from optimus_dl_b200.ops import rope as rope_ops
from optimus_dl_b200.ops.attention import attention_ref, build_doc_start, mask_from_doc_start

V = 97
MODELS = {
    "gpt2": dict(_name="gpt2", n_layer=2, n_head=4, n_embd=64, vocab_size=V, block_size=64),
    "llama2": dict(_name="llama2", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=V, sequence_length=64, multiple_of=8),
    "qwen3": dict(_name="qwen3", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, head_dim=32, vocab_size=V, sequence_length=64,
                  intermediate_size=96),
    "olmo3": dict(_name="olmo3", n_layer=2, n_head=4, n_kv_head=2, n_embd=64, vocab_size=V, sequence_length=64,
                  intermediate_size=96, layer_types=["sliding_attention", "full_attention"], sliding_window=8),
}


def _model(name, **over):
    torch.manual_seed(0)
    return build_model({**MODELS[name], **over}).eval()


@pytest.mark.parametrize("name", list(MODELS))
def test_future_tokens_never_change_earlier_logits(name):
    m = _model(name)
    x = torch.randint(0, V, (2, 20))
    y = x.clone()
    y[:, 12:] = torch.randint(0, V, (2, 8))
    a, b = m(x)["logits"], m(y)["logits"]
    assert torch.allclose(a[:, :12], b[:, :12], atol=1e-5)
    assert not torch.allclose(a[:, 12:], b[:, 12:], atol=1e-3)


@pytest.mark.parametrize("name", list(MODELS))
def test_samples_of_a_batch_do_not_see_each_other(name):
    m = _model(name)
    x = torch.randint(0, V, (3, 16))
    full = m(x)["logits"]
    for i in range(3):
        assert torch.allclose(full[i:i + 1], m(x[i:i + 1])["logits"], atol=1e-5)


@pytest.mark.parametrize("name", ["llama2", "qwen3", "olmo3"])
def test_padding_content_is_irrelevant_under_seq_lens(name):
    m = _model(name)
    x = torch.randint(0, V, (2, 18))
    lens = torch.tensor([18, 7])
    y = x.clone()
    y[1, 7:] = torch.randint(0, V, (11,))
    a = m(x, seq_lens=lens)["logits"]
    b = m(y, seq_lens=lens)["logits"]
    assert torch.allclose(a[0], b[0], atol=1e-5) and torch.allclose(a[1, :7], b[1, :7], atol=1e-5)
    assert torch.isfinite(a).all()                     # fully masked padding rows produce numbers, not NaN


def test_sliding_window_limits_the_receptive_field():
    # every layer windowed: position t sees t-w+1..t per layer, so two layers reach back 2 * (w - 1) tokens
    w = 4
    m = _model("qwen3", sliding_window=w)
    x = torch.randint(0, V, (1, 24))
    base = m(x)["logits"]
    far = x.clone()
    far[0, 3] = (far[0, 3] + 1) % V
    out = m(far)["logits"]
    reach = 3 + 2 * (w - 1)
    assert torch.allclose(out[:, reach + 1:], base[:, reach + 1:], atol=1e-5)
    assert not torch.allclose(out[:, 3:reach + 1], base[:, 3:reach + 1], atol=1e-4)
    unlimited = _model("qwen3")(far)["logits"] - _model("qwen3")(x)["logits"]
    assert unlimited[:, reach + 1:].abs().max() > 1e-4   # without the window the change travels on


def test_window_mask_matches_a_hand_written_mask():
    torch.manual_seed(0)
    B, T, H, hd, w = 2, 12, 2, 8, 5
    q, k, v = (torch.randn(B, T, H, hd) for _ in range(3))
    ds = build_doc_start(B, T, q.device)
    got = attention_ref(q.reshape(B * T, H, hd), k.reshape(B * T, H, hd), v.reshape(B * T, H, hd), ds,
                        window=w).reshape(B, T, H, hd)      # the op works on the flat token stream
    i = torch.arange(T)
    keep = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - w)
    s = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(hd)
    s = s.masked_fill(~keep, float("-inf"))
    want = torch.einsum("bhts,bshd->bthd", torch.softmax(s, -1), v)
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.equal(mask_from_doc_start(ds, window=w)[:T, :T], keep)


@pytest.mark.parametrize("name", ["llama2", "qwen3"])
def test_rotary_attention_depends_on_relative_positions_only(name):
    m = _model(name)
    x = torch.randint(0, V, (1, 14))
    pos = torch.arange(14)[None]
    a = m(x, position_ids=pos)["logits"]
    b = m(x, position_ids=pos + 17)["logits"]
    assert torch.allclose(a, m(x)["logits"], atol=1e-5)       # default positions are 0..T-1
    assert torch.allclose(a, b, atol=2e-4)                    # a common shift cancels in q.k
    c = m(x, position_ids=pos * 2)["logits"]
    assert not torch.allclose(a, c, atol=1e-3)


def test_rope_tables_scaling_variants_and_interleaved_pairs():
    f = rope_ops.precompute_freqs_cis(16, 32, theta=10000.0)
    assert f.shape == (32, 8, 2)
    assert torch.allclose(f[0, :, 0], torch.ones(8)) and torch.allclose(f[0, :, 1], torch.zeros(8))
    assert torch.allclose(f[5, 0], torch.tensor([math.cos(5.0), math.sin(5.0)]), atol=1e-6)   # lowest pair turns by 1 rad/token
    l3 = rope_ops.precompute_freqs_cis(16, 32, 10000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                          "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})
    assert torch.allclose(l3[:, 0], f[:, 0], atol=1e-6)       # high frequencies are kept
    assert not torch.allclose(l3[:, -1], f[:, -1], atol=1e-4)  # low frequencies are stretched
    yarn = rope_ops.precompute_freqs_cis(16, 32, 10000.0, {"rope_type": "yarn", "factor": 4.0,
                                                            "original_max_position_embeddings": 8})
    assert yarn.shape == f.shape and not torch.allclose(yarn, f, atol=1e-4)
    # pairs are (x0, x1), (x2, x3), ...: rotating by the table equals a complex multiplication per pair
    x = torch.randn(1, 32, 2, 16)
    got = rope_ops.rotate_ref(x, f)
    z = torch.view_as_complex(x.reshape(1, 32, 2, 8, 2)) * torch.view_as_complex(f.contiguous())[None, :, None]
    assert torch.allclose(got, torch.view_as_real(z).flatten(-2), atol=1e-6)
    assert torch.allclose(rope_ops.rotate_ref(got, f, inverse=True), x, atol=1e-5)


@pytest.mark.parametrize("name", ["llama2", "olmo3"])
def test_packed_batch_gradients_equal_the_sum_over_separate_documents(name):
    m = _model(name).train()
    a, b = torch.randint(0, V, (1, 9)), torch.randint(0, V, (1, 13))

    def grads(run):
        m.zero_grad()
        run().backward()
        return {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}

    sep = grads(lambda: m(a)["logits"].float().logsumexp(-1).sum() + m(b)["logits"].float().logsumexp(-1).sum())
    packed = torch.cat([a, b], 1)
    pos = torch.cat([torch.arange(9), torch.arange(13)])[None]
    doc = torch.cat([torch.zeros(9), torch.ones(13)])[None].long()
    pk = grads(lambda: m(packed, document_ids=doc, position_ids=pos)["logits"].float().logsumexp(-1).sum())
    assert sep.keys() == pk.keys()
    for n in sep:
        assert torch.allclose(sep[n], pk[n], atol=2e-4, rtol=1e-3), n


def test_gqa_equals_full_heads_with_repeated_kv():
    torch.manual_seed(0)
    B, T, Hq, Hk, hd = 1, 10, 4, 2, 8
    q = torch.randn(B, T, Hq, hd)
    k, v = torch.randn(B, T, Hk, hd), torch.randn(B, T, Hk, hd)
    ds = build_doc_start(B, T, q.device)
    q, k, v = q[0], k[0], v[0]
    grouped = attention_ref(q, k, v, ds)
    full = attention_ref(q, k.repeat_interleave(2, dim=1), v.repeat_interleave(2, dim=1), ds)
    assert torch.allclose(grouped, full, atol=1e-6)


def test_sequence_longer_than_the_configured_length_is_refused():
    m = _model("llama2")
    with pytest.raises(AssertionError):
        m(torch.randint(0, V, (1, 65)))


def test_doc_start_masks_equal_the_visibility_predicate():
    from optimus_dl_b200.models.blocks.attention import attention_mask_fn

    B, T, w = 2, 10, 4
    docs = torch.tensor([[0, 0, 0, 1, 1, 1, 1, 2, 2, 2], [3, 3, 3, 3, 3, 3, 3, 3, 3, 3]])
    q = torch.arange(T)[:, None].expand(T, T)
    k = torch.arange(T)[None, :].expand(T, T)
    for window in (None, w):
        got = mask_from_doc_start(build_doc_start(B, T, docs.device, document_ids=docs), window=window)
        for b in range(B):
            want = attention_mask_fn(b, None, q, k, window_size=window, document_ids=docs)
            assert torch.equal(got[b * T:(b + 1) * T, b * T:(b + 1) * T], want), (window, b)
        assert not got[:T, T:].any() and not got[T:, :T].any()      # samples of a batch never see each other
    lens = torch.tensor([10, 6])
    pred = torch.stack([attention_mask_fn(b, None, q, k, seq_lens=lens) for b in range(B)])
    assert pred[1, 5, :6].all() and not pred[1, 7].any() and not pred[1, :, 6:].any() and pred[0].equal(k <= q)


def test_attention_dropout_acts_on_the_probabilities_in_training_only():
    """GPT-2 with ``dropout > 0``: the attention block drops probabilities (and residual outputs) while training,
    and is exactly the dropout-free block in evaluation mode
    (optimus_dl/modules/model/blocks/attention.py:133-134, 528)."""
    from optimus_dl_b200.ops.attention import attention_sdpa_rows

    B, T, Hq, Hk, hd = 2, 12, 4, 2, 16
    torch.manual_seed(1)
    q, k, v = torch.randn(B, T, Hq, hd), torch.randn(B, T, Hk, hd), torch.randn(B, T, Hk, hd)
    docs = torch.tensor([[0] * 5 + [1] * 7, [2] * 12])
    ds = build_doc_start(B, T, q.device, document_ids=docs)
    for window in (None, 3):
        rows = attention_sdpa_rows(q, k, v, ds, window, 1.0 / math.sqrt(hd))
        flat = attention_ref(q.reshape(B * T, Hq, hd), k.reshape(B * T, Hk, hd), v.reshape(B * T, Hk, hd), ds, window)
        assert torch.allclose(rows.reshape(B * T, Hq, hd), flat, atol=1e-5)
    m = _model("gpt2", dropout=0.3)
    plain = _model("gpt2")
    plain.load_state_dict(m.state_dict())
    x = torch.randint(0, V, (2, 16))
    assert torch.allclose(m(x)["logits"], plain(x)["logits"], atol=1e-6)
    att = m.transformer.h[0].attn
    assert att.attn_dropout.p == 0.3 and att.resid_dropout.p == 0.3
    att.train()
    h = torch.randn(2, 16, 64)
    torch.manual_seed(5)
    a = att(h)
    torch.manual_seed(6)
    b = att(h)
    assert not torch.allclose(a, b) and torch.isfinite(a).all()
    att.resid_dropout.p = 0.0                      # what is left is the dropout inside the attention product
    torch.manual_seed(5)
    c = att(h)
    torch.manual_seed(6)
    d = att(h)
    assert not torch.allclose(c, d)
