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


def _engine_setup(extra_transforms=(), fsdp=None, opt_cfg=None):
    from optimus_dl_b200.criterion import build_criterion
    from optimus_dl_b200.model_transforms import build_model_transform
    from optimus_dl_b200.optim import build_optimizer

    ref, gpu = _models()
    dev = torch.device("cuda", 0)
    for t in extra_transforms:
        gpu = build_model_transform(t).apply(gpu, collective=None, device=dev)
    gpu = build_model_transform(dict({"_name": "fully_shard"}, **(fsdp or {}))).apply(gpu, collective=None, device=dev)
    crit = build_criterion({"_name": "cross_entropy"})
    opt = build_optimizer(dict({"_name": "adamw", "lr": 1e-3, "betas": [0.9, 0.95], "weight_decay": 0.1}, **(opt_cfg or {})),
                          params=gpu.make_parameter_groups())
    return ref, gpu, crit, opt


def test_failed_wait_stops_the_step_and_keeps_the_weights():
    """A kernel whose bounded wait runs out leaves its code in the status word. The optimizer step of that
    iteration must not be committed (the update kernels skip their writes) and the error must surface from the
    training step itself: at ``verify()`` at once, or at the next ``step()``."""
    from optimus_dl_b200.ops import _lib, gemm

    _, gpu, crit, opt = _engine_setup()
    eng = gpu._sharding_engine
    ids = torch.randint(0, 1000, (2, 65), device="cuda")

    def one_step():
        opt.zero_grad()
        loss, _ = crit(gpu, {"input_ids": ids})
        loss.backward()
        opt.step()
        return loss

    one_step()
    eng.verify()
    masters = [g.master.clone() for g in eng.groups]
    moments = [g.exp_avg.clone() for g in eng.groups]
    # make a wait run out: a GEMM whose operand flags nothing ever sets (bounded at two seconds)
    a = torch.randn(128, 128, device="cuda").bfloat16()
    b = torch.randn(256, 128, device="cuda").bfloat16()
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    gemm.gemm(a, b, b_flags=flags, flag_rows=128, flag_value=1, tile_order=1)
    one_step()                      # runs with the status word set
    torch.cuda.synchronize()
    for g, m0, e0 in zip(eng.groups, masters, moments):
        assert torch.equal(g.master, m0) and torch.equal(g.exp_avg, e0), "a step with a failed wait was committed"
    with pytest.raises(_lib.KernelError, match="flag wait timed out"):
        one_step()                  # the deferred read of the previous step raises before anything else happens
    _lib.check_status()             # ... and clears the word: training can go on
    one_step()
    eng.verify()
    assert not torch.equal(eng.groups[0].master, masters[0])


def test_eight_micro_batches_accumulate_in_fp32():
    """Gradients of micro-batches are summed in the fp32 gradient shards: after 8 micro-batches the shard equals
    the fp32 sum of the 8 single-micro-batch gradients exactly (an accumulator that rounded to bf16 in between
    would not), and it tracks an fp32 run of the model."""
    from optimus_dl_b200.model_transforms.distributed import accumulation_context
    from optimus_dl_b200.ops import _lib

    ref, gpu, crit, opt = _engine_setup(opt_cfg={"weight_decay": 0.0})
    opt.set_max_norm(1e9)            # keeps the update out of the reduce kernel, so the gradient shards can be read
    eng = gpu._sharding_engine
    torch.manual_seed(3)
    batches = [torch.randint(0, 1000, (2, 65)) for _ in range(8)]
    crit.grad_scale = 1.0 / 8
    singles = []
    for b in batches:
        opt.zero_grad()
        with accumulation_context(gpu, False):
            (crit(gpu, {"input_ids": b.cuda()})[0] / 8).backward()
        torch.cuda.synchronize()
        singles.append([g.grad_shard.clone() for g in eng.groups])
    opt.zero_grad()
    for i, b in enumerate(batches):
        with accumulation_context(gpu, i == len(batches) - 1):
            (crit(gpu, {"input_ids": b.cuda()})[0] / 8).backward()
    torch.cuda.synchronize()
    crit.grad_scale = 1.0
    _lib.check_status()
    for gi, g in enumerate(eng.groups):
        expect = torch.zeros_like(g.grad_shard)
        for s_ in singles:
            expect += s_[gi]
        assert torch.equal(g.grad_shard, expect), f"group {g.name}: accumulation is not an exact fp32 sum"
    for b in batches:
        (crit(ref, {"input_ids": b})[0] / 8).backward()
    names = dict(ref.named_parameters())
    for name, g, inf in eng.named_sharded_state():
        got = g.local_shard(inf, g.grad_shard).float().cpu()
        want = names[name].grad.reshape(got.shape)
        assert ((got - want).abs().max() / (want.abs().max() + 1e-12)).item() < 0.12, name
    opt.step()
    eng.verify()


def test_activation_checkpointing_on_the_kernel_path():
    """`activation_checkpoint` + `fully_shard`: the recomputation re-enters the engine's forward hooks and the
    in-place rotary kernel inside the backward pass; loss and updated weights equal the run without it."""
    from optimus_dl_b200.ops import _lib

    runs = []
    for transforms in ((), ({"_name": "activation_checkpoint", "layer_classes": ["LlamaBlock"]},)):
        _, gpu, crit, opt = _engine_setup(extra_transforms=transforms)
        torch.manual_seed(4)
        losses = []
        for _ in range(3):
            ids = torch.randint(0, 1000, (2, 97), device="cuda")
            opt.zero_grad()
            loss, _ = crit(gpu, {"input_ids": ids})
            loss.backward()
            opt.step()
            losses.append(loss.item())
        torch.cuda.synchronize()
        _lib.check_status()
        runs.append((losses, [g.master.clone() for g in gpu._sharding_engine.groups]))
    (l0, m0), (l1, m1) = runs
    assert l0 == l1, (l0, l1)
    for a, b in zip(m0, m1):
        assert torch.equal(a, b)
