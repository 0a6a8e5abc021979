"""End-to-end checks of the kernel path against fp32 PyTorch on the same weights."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(_name="llama2", n_layer=2, n_head=8, n_kv_head=2, n_embd=256, intermediate_size=768, vocab_size=1000,
           sequence_length=256, tie_word_embeddings=False)


def _models():
    from optimus_dl_b200.models import build_model

    torch.manual_seed(0)
    ref = build_model(CFG)  # fp32 on CPU
    gpu = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    return ref, gpu


def test_llama_forward_backward_matches_fp32():
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.ops import _lib

    ref, gpu = _models()
    crit = build_criterion({"_name": "cross_entropy"})
    ids = torch.randint(0, 1000, (2, 129))
    doc = torch.tensor([[0] * 40 + [1] * 89, [0] * 129])
    l_ref, _ = crit(ref, {"input_ids": ids, "document_ids": doc})
    l_ref.backward()
    l_gpu, _ = crit(gpu, {"input_ids": ids.cuda(), "document_ids": doc.cuda()})
    l_gpu.backward()
    _lib.check_status()
    assert abs(l_ref.item() - l_gpu.item()) < 3e-2, (l_ref.item(), l_gpu.item())
    for (n, p), (_, q) in zip(ref.named_parameters(), gpu.named_parameters()):
        a, b = q.grad.float().cpu(), p.grad
        denom = b.abs().max().item() + 1e-6
        assert (a - b).abs().max().item() / denom < 0.12, f"grad mismatch for {n}"


def test_sharded_engine_single_gpu_tracks_adamw():
    """World of one: flat buffers + fused reduce/update kernel versus torch AdamW on fp32 weights."""
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.model_transforms import build_model_transform
    from optimus_dl_b200.optim import build_optimizer
    from optimus_dl_b200.ops import _lib

    ref, gpu = _models()
    dev = torch.device("cuda", 0)
    gpu = build_model_transform({"_name": "fully_shard"}).apply(gpu, collective=None, device=dev)
    crit = build_criterion({"_name": "cross_entropy"})
    opt = build_optimizer({"_name": "adamw", "lr": 1e-3, "betas": [0.9, 0.95], "weight_decay": 0.1},
                          params=gpu.make_parameter_groups())
    groups = ref.make_parameter_groups()
    ref_opt = torch.optim.AdamW([dict(g, params=[p for _, p in g["params"]]) for g in groups], lr=1e-3,
                                betas=(0.9, 0.95), weight_decay=0.1)
    torch.manual_seed(1)
    losses_ref, losses_gpu = [], []
    for step in range(4):
        ids = torch.randint(0, 1000, (2, 65))
        ref_opt.zero_grad()
        lr_, _ = crit(ref, {"input_ids": ids})
        lr_.backward()
        ref_opt.step()
        opt.zero_grad()
        lg, _ = crit(gpu, {"input_ids": ids.cuda()})
        lg.backward()
        opt.step()
        losses_ref.append(lr_.item())
        losses_gpu.append(lg.item())
    torch.cuda.synchronize()
    _lib.check_status()
    for a, b in zip(losses_ref, losses_gpu):
        assert abs(a - b) < 5e-2, (losses_ref, losses_gpu)
    assert losses_gpu[-1] < losses_gpu[0]
    # fused QKV view: the three projection weights are adjacent in the flat buffer
    attn = gpu.transformer.h[0].attn
    from optimus_dl_b200.ops.linear import _adjacent

    assert _adjacent([attn.wq.weight, attn.wk.weight, attn.wv.weight])
    assert _adjacent([attn.wq.weight.main_grad, attn.wk.weight.main_grad, attn.wv.weight.main_grad])


def test_grad_accumulation_and_clipping_two_phase():
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.model_transforms import build_model_transform
    from optimus_dl_b200.model_transforms.distributed import accumulation_context
    from optimus_dl_b200.optim import build_optimizer
    from optimus_dl_b200.ops import _lib

    ref, gpu = _models()
    dev = torch.device("cuda", 0)
    gpu = build_model_transform({"_name": "fully_shard"}).apply(gpu, collective=None, device=dev)
    crit = build_criterion({"_name": "cross_entropy"})
    opt = build_optimizer({"_name": "adamw", "lr": 1e-3, "weight_decay": 0.0}, params=gpu.make_parameter_groups())
    opt.set_max_norm(0.5)
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.0)
    torch.manual_seed(2)
    batches = [torch.randint(0, 1000, (2, 65)) for _ in range(2)]
    ref_opt.zero_grad()
    for b in batches:
        (crit(ref, {"input_ids": b})[0] / 2).backward()
    norm_ref = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
    ref_opt.step()
    opt.zero_grad()
    crit.grad_scale = 0.5
    for i, b in enumerate(batches):
        with accumulation_context(gpu, i == len(batches) - 1):
            (crit(gpu, {"input_ids": b.cuda()})[0] / 2).backward()
    opt.step()
    torch.cuda.synchronize()
    _lib.check_status()
    assert abs(opt.grad_norm().item() - norm_ref.item()) / norm_ref.item() < 0.05, (opt.grad_norm().item(), norm_ref.item())
    l1 = crit(ref, {"input_ids": batches[0]})[0].item()
    crit.grad_scale = 1.0
    l2 = crit(gpu, {"input_ids": batches[0].cuda()})[0].item()
    assert abs(l1 - l2) < 5e-2
