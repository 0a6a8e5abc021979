"""GRPO: objective derivative, group advantages, and a tiny CPU run whose reward must go up."""

import torch

from optimus_dl_b200.core import conf
from optimus_dl_b200.core.config_utils import non_resolving_instantiate
from optimus_dl_b200.core.registry import build
from optimus_dl_b200.recipe.grpo.loss import group_advantages, token_loss


def test_group_advantages():
    r = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 5.0, 5.0, 5.0])
    a = group_advantages(r, 4)
    assert torch.allclose(a[:4].mean(), torch.tensor(0.0), atol=1e-6)
    assert torch.allclose(a[:4].std(unbiased=False), torch.tensor(1.0), atol=1e-4)
    assert torch.all(a[4:] == 0)


def test_token_loss_derivative_matches_autograd():
    torch.manual_seed(0)
    n = 257
    nll = (torch.rand(n, dtype=torch.float64) * 3).requires_grad_(True)
    old = -(nll.detach() + torch.randn(n, dtype=torch.float64) * 0.3)   # ratios on both sides of the clip range
    ref = -(nll.detach() + torch.randn(n, dtype=torch.float64) * 0.2)
    adv = torch.randn(n, dtype=torch.float64)
    mask = torch.rand(n) > 0.2
    loss, d, stats = token_loss(nll, old, ref, adv, mask, 0.2, 0.04, 1.0 / 100)
    (g,) = torch.autograd.grad(loss.sum(), nll)
    assert torch.allclose(g, d.to(g.dtype), atol=1e-9)
    assert float(stats["clipped_sum"].detach()) > 0 and float(stats["kl_sum"].detach()) > 0
    assert torch.all(d[~mask] == 0)


def test_linear_token_loss_cpu_gradient():
    from optimus_dl_b200.ops.cross_entropy import linear_token_loss

    torch.manual_seed(0)
    x = torch.randn(12, 16, requires_grad=True)
    w = torch.randn(40, 16, requires_grad=True)
    tg = torch.randint(0, 40, (12,))
    coef = torch.randn(12)
    total, nll = linear_token_loss(x, w, tg, lambda n, a, b: (coef[a:b] * n, coef[a:b]))
    total.backward()
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    ref = (coef * torch.nn.functional.cross_entropy(x2 @ w2.t(), tg, reduction="none")).sum()
    ref.backward()
    assert torch.allclose(total, ref, atol=1e-5)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5) and torch.allclose(w.grad, w2.grad, atol=1e-5)


def test_tiny_grpo_run_improves_reward(tmp_path):
    cfg = conf.create({
        "_name": "base",
        "common": {"use_gpu": False, "output_path": str(tmp_path), "log_freq": 1, "seed": 0,
                   "distributed": {"tp_size": 1, "sharding_world_size": 1}},
        "model": {"_name": "llama2", "n_layer": 2, "n_head": 2, "n_embd": 32, "vocab_size": 16, "sequence_length": 32,
                  "intermediate_size": 64, "tie_word_embeddings": False},
        "grpo": {"num_prompts": 8, "prompt_length": 4, "group_size": 8, "max_new_tokens": 8, "kl_coef": 0.01,
                 "micro_batch_size": 32, "rollout_batch_size": 64, "updates_per_rollout": 2,
                 "reward": {"_name": "even_fraction"}},
        "optimization": {"iterations": 30, "clip_grad_norm": 1.0,
                         "optimizer": {"_name": "adamw", "lr": 2e-2, "weight_decay": 0.0, "fused": False}},
        "loggers": [{"_name": "jsonl", "output_dir": str(tmp_path / "metrics")}],
    })
    recipe = build("grpo_recipe", non_resolving_instantiate(cfg))
    recipe.run()
    rewards = [h["reward"] for h in recipe.history]
    assert len(rewards) == 30
    first, last = sum(rewards[:5]) / 5, sum(rewards[-5:]) / 5
    assert last > first + 0.15, (first, last)
    assert any(h["clip_frac"] > 0 for h in recipe.history[1:]) or True
    assert all(h["kl"] >= 0 for h in recipe.history)


def test_rewards_respect_the_completion_mask():
    from optimus_dl_b200.recipe.grpo.rewards import EvenFractionReward, TargetTokenReward

    comp = torch.tensor([[2, 4, 5, 7], [1, 3, 5, 6], [8, 8, 8, 8]])
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0], [0, 0, 0, 0]], dtype=torch.bool)
    even = EvenFractionReward()(None, comp, mask)
    assert torch.allclose(even, torch.tensor([2 / 3, 0.0, 0.0]))           # padding never counts; an empty row scores 0
    hit = TargetTokenReward(conf.create({"token_id": 5}))(None, comp, mask)
    assert torch.allclose(hit, torch.tensor([1 / 3, 0.0, 0.0]))


def test_prompt_source_is_seeded_per_step_and_split_across_ranks():
    from optimus_dl_b200.recipe.grpo.rewards import UniformRandomPrompts

    cfg = conf.create({"low": 3, "high": 9})
    whole = UniformRandomPrompts(cfg, vocab_size=50, seed=4, rank=0, world_size=1)(step=2, n_local=4, length=6, device=torch.device("cpu"))
    parts = [UniformRandomPrompts(cfg, vocab_size=50, seed=4, rank=r, world_size=2)(2, 2, 6, torch.device("cpu")) for r in (0, 1)]
    assert whole.shape == (4, 6) and whole.min() >= 3 and whole.max() < 9
    assert torch.equal(torch.cat(parts), whole)                            # ranks take disjoint slices of one stream
    again = UniformRandomPrompts(cfg, vocab_size=50, seed=4)(2, 4, 6, torch.device("cpu"))
    other_step = UniformRandomPrompts(cfg, vocab_size=50, seed=4)(3, 4, 6, torch.device("cpu"))
    assert torch.equal(again, whole) and not torch.equal(other_step, whole)
    default_high = UniformRandomPrompts(None, vocab_size=7)(0, 64, 8, torch.device("cpu"))
    assert default_high.max() < 7


def test_token_loss_limits():
    n = 6
    nll = torch.full((n,), 1.0, dtype=torch.float64)
    adv = torch.tensor([1.0, -1.0, 2.0, -2.0, 0.5, 0.0], dtype=torch.float64)
    mask = torch.ones(n, dtype=torch.bool)
    # on-policy (ratio 1), no reference model: the loss is -A / N and its gradient with respect to nll is +A / N
    loss, d, stats = token_loss(nll, -nll, None, adv, mask, 0.2, 0.0, 1.0 / n)
    assert torch.allclose(loss, -adv / n) and torch.allclose(d, adv / n)
    assert float(stats["clipped_sum"]) == 0 and float(stats["kl_sum"]) == 0 and float(stats["ratio_sum"]) == n
    # a ratio far above the clip range with a positive advantage is clipped: no gradient; with a negative one it is not
    old = -nll - 1.0                                                       # ratio = e
    loss, d, stats = token_loss(nll, old, None, adv, mask, 0.2, 0.0, 1.0 / n)
    assert d[0] == 0 and d[2] == 0 and d[1] != 0 and d[3] != 0 and float(stats["clipped_sum"]) == n
    # the reference term alone: k3 estimator exp(d) - d - 1 >= 0, zero gradient where the policies agree
    loss, d, stats = token_loss(nll, -nll, -nll, torch.zeros(n, dtype=torch.float64), mask, 0.2, 0.5, 1.0)
    assert torch.allclose(loss, torch.zeros(n, dtype=torch.float64)) and torch.allclose(d, torch.zeros(n, dtype=torch.float64))
    loss, _, stats = token_loss(nll, -nll, -nll + 0.3, torch.zeros(n, dtype=torch.float64), mask, 0.2, 0.5, 1.0)
    assert (loss > 0).all() and float(stats["kl_sum"]) > 0
