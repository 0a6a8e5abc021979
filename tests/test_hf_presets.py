"""Weight conversion from Hugging Face models: logits of the converted model must match transformers' own
implementation (tiny random models built offline from configs)."""

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _compare(hf_model, ours, vocab):
    ids = torch.randint(0, vocab, (2, 24), generator=torch.Generator().manual_seed(0))
    with torch.no_grad():
        ref = hf_model(ids).logits.float()
        got = ours(ids)["logits"].float()
    err = (ref - got).abs().max().item()
    assert err < 2e-4, err


def test_permute_rope_weight_layout():
    from optimus_dl_b200.models.presets.utils import permute_rope_weight

    w = torch.arange(2 * 8).float().reshape(16, 1)   # 2 heads, head_dim 8
    p = permute_rope_weight(w, 2, 8).flatten().tolist()
    assert p[:8] == [0, 4, 1, 5, 2, 6, 3, 7] and p[8:] == [8, 12, 9, 13, 10, 14, 11, 15]
    v = permute_rope_weight(torch.arange(8).float(), 2, 8).tolist()
    assert v == [0, 4, 1, 5, 2, 6, 3, 7]


def test_llama_conversion_matches_transformers():
    from optimus_dl_b200.models.presets.hf_llama import HFLlamaConfig, llama_from_hf

    torch.manual_seed(0)
    hf_cfg = transformers.LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                      rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
                                      attn_implementation="eager")
    hf = transformers.LlamaForCausalLM(hf_cfg).eval()
    ours = llama_from_hf(HFLlamaConfig(), hf_cfg, hf.state_dict()).eval()
    assert ours.config.n_kv_head == 2 and ours.config.intermediate_size == 112
    _compare(hf, ours, 128)


def test_qwen3_conversion_matches_transformers():
    if not hasattr(transformers, "Qwen3ForCausalLM"):
        pytest.skip("transformers without Qwen3")
    from optimus_dl_b200.models.presets.hf_qwen3 import HFQwen3Config, qwen3_from_hf

    torch.manual_seed(0)
    hf_cfg = transformers.Qwen3Config(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                      max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=1e6,
                                      tie_word_embeddings=True, attention_bias=False, attn_implementation="eager")
    hf = transformers.Qwen3ForCausalLM(hf_cfg).eval()
    for name, p in hf.named_parameters():   # non-trivial norm weights so that a wrong permutation shows
        if "norm" in name:
            torch.nn.init.normal_(p, mean=1.0, std=0.2)
    ours = qwen3_from_hf(HFQwen3Config(), hf_cfg, hf.state_dict()).eval()
    assert ours.config.head_dim == 32 and ours.transformer.wte.weight is ours.lm_head.weight
    _compare(hf, ours, 128)


def test_olmo3_conversion_matches_transformers():
    if not hasattr(transformers, "Olmo3ForCausalLM"):
        pytest.skip("transformers without Olmo3")
    from optimus_dl_b200.models.presets.hf_olmo3 import HFOlmo3Config, olmo3_from_hf

    torch.manual_seed(0)
    hf_cfg = transformers.Olmo3Config(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                      rms_norm_eps=1e-6, sliding_window=8,
                                      layer_types=["sliding_attention", "sliding_attention", "sliding_attention",
                                                   "full_attention"], tie_word_embeddings=False,
                                      attn_implementation="eager")
    hf = transformers.Olmo3ForCausalLM(hf_cfg).eval()
    for name, p in hf.named_parameters():
        if "norm" in name:
            torch.nn.init.normal_(p, mean=1.0, std=0.2)
    ours = olmo3_from_hf(HFOlmo3Config(), hf_cfg, hf.state_dict()).eval()
    _compare(hf, ours, 128)
