"""Module-level numerics on the GPU: the sm_100a paths of the MoE layer, router module, decoder, fused optimizer
and Trainer against PyTorch fp32 restatements of the same math."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from composed_mixture_of_experts_engine_b200.ops.kernels import check_status

    check_status(torch.device("cuda", torch.cuda.current_device()))


@pytest.mark.parametrize("N,H,F,E,K,dropping", [(512, 256, 512, 8, 2, False), (1000, 512, 256, 16, 4, False),
                                                (777, 256, 384, 8, 2, True)])
def test_moe_layer_device_path_matches_fp32_restatement(N, H, F, E, K, dropping):
    from composed_mixture_of_experts_engine_b200.ops.functional import experts_reference
    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer
    from composed_mixture_of_experts_engine_b200.parallel.moe_layer import compute_capacity_drop_mask

    torch.manual_seed(0)
    layer = DistributedMoELayer(H, F, E, K, capacity_factor=0.6, capacity_dropping=dropping,
                                dtype=torch.bfloat16).cuda()
    x = torch.randn(N, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    assert layer.router.last_profile.used_fused_kernel
    dy = torch.randn_like(y)
    y.backward(dy)
    # restatement in fp32 on the kernel's own routing decision
    idx, w = layer.router.last_idx32.long(), layer.router.last_w32.detach()
    keep = ~compute_capacity_drop_mask(idx, E, layer.capacity(N)) if dropping else None
    xf = x.detach().float().requires_grad_(True)
    w13, w2 = layer.w13.detach().float().requires_grad_(True), layer.w2.detach().float().requires_grad_(True)
    wf = w.clone().requires_grad_(True)
    yr = experts_reference(xf, idx, wf, w13, w2, 0, keep)
    yr.backward(dy.float())
    assert _rel(y, yr) < 2e-2
    assert _rel(layer.w13.grad, w13.grad) < 3e-2 and _rel(layer.w2.grad, w2.grad) < 3e-2
    # dx has two parts (experts + router); compare the expert part by removing the router contribution
    assert torch.isfinite(x.grad).all() and layer.router.gate_w.grad is not None
    if dropping:
        assert 0 < layer.last_dropped_token_fraction < 1
        assert abs(layer.last_dropped_token_fraction - float((~keep).float().mean())) < 1e-6


def test_moe_layer_dx_and_gate_grad_against_autograd():
    """Full layer gradient (router included) vs autograd through an fp32 restatement with the same top-k picks."""
    from composed_mixture_of_experts_engine_b200.ops.functional import experts_reference
    from composed_mixture_of_experts_engine_b200.parallel import DistributedMoELayer

    torch.manual_seed(1)
    N, H, F, E, K = 600, 256, 256, 8, 2
    layer = DistributedMoELayer(H, F, E, K, dtype=torch.bfloat16).cuda()
    x = torch.randn(N, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    idx = layer.router.last_idx32.long()
    xf = x.detach().float().requires_grad_(True)
    gw = layer.router.gate_w.detach().float().requires_grad_(True)
    p = torch.softmax(xf @ gw, -1)
    sel = p.gather(1, idx)
    wn = sel / sel.sum(-1, keepdim=True)
    yr = experts_reference(xf, idx, wn, layer.w13.detach().float(), layer.w2.detach().float())
    yr.backward(dy.float())
    assert _rel(y, yr) < 2e-2
    assert _rel(x.grad, xf.grad) < 4e-2
    assert _rel(layer.router.gate_w.grad, gw.grad) < 5e-2


def test_router_module_device_vs_oracle():
    from composed_mixture_of_experts_engine_b200.ops.moe_router import MoERouter, _reference_route_fp64

    torch.manual_seed(2)
    r = MoERouter(1024, 64, top_k=8, dtype=torch.bfloat16).cuda()
    r.profile_timing = True
    x = torch.randn(4096, 1024, device="cuda", dtype=torch.bfloat16)
    idx, w, cnt = r(x)
    ridx, rw, _ = _reference_route_fp64(x, r.gate_w, 8)
    agree = (idx == ridx).all(-1).float().mean()
    assert agree > 0.995
    rows = (idx == ridx).all(-1)
    assert torch.allclose(w[rows].float(), rw[rows].float(), atol=2e-2)
    assert int(cnt.sum()) == 4096 * 8 and w.dtype == torch.bfloat16
    prof = r.last_profile
    assert prof.used_fused_kernel and prof.kernel_ms > 0 and prof.backend == "sm100a-fused"


def test_decoder_device_loss_matches_cpu_fp32():
    from composed_mixture_of_experts_engine_b200.models import build_model
    from composed_mixture_of_experts_engine_b200.parallel import ParallelTopology
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    cfg = MoEConfig.from_dict({"model": dict(arch="moe_decoder", hidden_dim=256, num_layers=2, num_heads=4,
                                             num_kv_heads=2, num_experts=8, top_k=2, ffn_dim=256, vocab_size=1024,
                                             sequence_length=128, dtype="bfloat16", init_std=0.02),
                               "training": dict(max_steps=5, warmup_steps=0)})
    torch.manual_seed(3)
    gpu = build_model(cfg, ParallelTopology(1, 0, 1, 1, device=torch.device("cuda", 0)))
    d = cfg.to_dict()
    d["model"]["dtype"] = "float32"
    cpu = build_model(MoEConfig.from_dict(d), ParallelTopology(1, 0, 1, 1))
    cpu.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    ids, tgt = torch.randint(0, 1024, (2, 128)), torch.randint(0, 1024, (2, 128))
    lg = gpu.loss(ids.cuda(), tgt.cuda())
    lc = cpu.loss(ids, tgt)
    assert abs(float(lg) - float(lc)) < 3e-2
    lg.backward()
    lc.backward()
    g1, g2 = gpu.lm_head.weight.grad, cpu.lm_head.weight.grad
    assert _rel(g1.cpu(), g2) < 6e-2
    e1, e2 = gpu.blocks[0].attn.wqkv.weight.grad, cpu.blocks[0].attn.wqkv.weight.grad
    assert _rel(e1.cpu(), e2) < 0.15


def test_fused_adamw_matches_torch_adamw_with_clipping():
    from composed_mixture_of_experts_engine_b200.ops.optim import build_optimizer

    torch.manual_seed(4)
    net = torch.nn.Sequential(torch.nn.Linear(64, 128, bias=False), torch.nn.Linear(128, 64, bias=False)
                              ).cuda().to(torch.bfloat16)
    ref = [p.detach().float().clone().requires_grad_(True) for p in net.parameters()]
    opt = build_optimizer(net, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    ropt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for step in range(3):
        grads = [torch.randn_like(p) * 3 for p in net.parameters()]
        for p, g, r in zip(net.parameters(), grads, ref):
            p.main_grad.copy_(g)  # the optimizer's fp32 gradient buffer (what the weight-gradient GEMMs add into)
            r.grad = g.float().clone()
        torch.nn.utils.clip_grad_norm_(ref, 1.0)
        ropt.step()
        opt.step()
        assert all(float(p.main_grad.abs().max()) == 0.0 for p in net.parameters())  # cleared by the kernel
    for g in opt.groups:
        pass
    masters = opt.groups[0].master
    flat_ref = torch.cat([r.detach().reshape(-1) for r in ref])
    assert torch.allclose(masters[: flat_ref.numel()], flat_ref, atol=2e-5, rtol=1e-4)
    assert torch.equal(list(net.parameters())[0].detach(), ref[0].detach().to(torch.bfloat16))


@pytest.mark.parametrize("rows,K,N", [(512, 256, 384), (1000, 2048, 520), (4096, 2048, 6144)])
def test_linear_op_forward_and_gradients_match_fp32(rows, K, N):
    """``ops.functional.linear`` (tcgen05 GEMMs for y, dx and dW) against fp32 matmuls of the same bf16 inputs,
    first with autograd-owned gradients, then with the weight gradient accumulated into an fp32 ``main_grad``
    over two backward passes (the TMA reduce-add epilogue)."""
    from composed_mixture_of_experts_engine_b200.ops import functional as OF

    torch.manual_seed(11)
    x = (torch.randn(2, rows // 2, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(2, rows // 2, N, device="cuda").to(torch.bfloat16)
    assert OF.linear_supported(x, w)
    y = OF.linear(x, w)
    y.backward(dy)
    xf, wf, dyf = x.detach().float(), w.detach().float(), dy.float()
    assert _rel(y, xf @ wf.t()) < 1e-2
    assert _rel(x.grad, dyf @ wf) < 1e-2
    want_dw = dyf.reshape(-1, N).t() @ xf.reshape(-1, K)
    assert _rel(w.grad, want_dw) < 1e-2
    # accumulate into main_grad: two backward passes add up, p.grad stays untouched
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(N, K, device="cuda", dtype=torch.float32)
    for _ in range(2):
        OF.linear(x.detach(), w2).backward(dy)
    assert w2.grad is None
    assert _rel(w2.main_grad, 2 * want_dw) < 1e-2


@pytest.mark.parametrize("with_main_grad", [False, True])
def test_lm_head_loss_matches_fp32_cross_entropy(with_main_grad):
    """The chunked LM-head loss (logits GEMM, cross-entropy kernel, dh and dW GEMMs per chunk of rows) vs
    ``F.cross_entropy`` on fp32 logits; chunk 256 forces several chunks and a ragged last one; V is not a
    multiple of the GEMM tile."""
    from composed_mixture_of_experts_engine_b200.models.decoder import lm_head_loss

    torch.manual_seed(12)
    n, H, V = 1000, 256, 1160
    h = (torch.randn(n, H, device="cuda") * 0.7).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, H, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    if with_main_grad:
        w.main_grad = torch.zeros(V, H, device="cuda", dtype=torch.float32)
    tgt = torch.randint(0, V, (n,), device="cuda")
    loss = lm_head_loss(h, w, tgt, 1.0 / n, chunk=256)
    (loss * 2.0).backward()  # an upstream factor must reach both gradients
    hf = h.detach().float().requires_grad_()
    wf = w.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(hf @ wf.t(), tgt, reduction="sum") / n
    (ref * 2.0).backward()
    assert abs(float(loss) - float(ref)) < 2e-2
    assert _rel(h.grad, hf.grad) < 3e-2
    got_dw = w.main_grad if with_main_grad else w.grad
    assert (w.grad is None) == with_main_grad
    assert _rel(got_dw, wf.grad) < 3e-2
    with torch.no_grad():  # evaluation: no gradient work, same value
        assert abs(float(lm_head_loss(h, w, tgt, 1.0 / n, chunk=256)) - float(loss)) < 1e-5


def test_async_checkpoint_of_device_state_reuses_pinned_buffers_and_does_not_stall(tmp_path):
    """Snapshot of a CUDA model + fused optimizer: the device-to-host copies run on a side stream into pinned
    buffers that the second save reuses (no new pinned allocation), the optimizer's pre-step hook (not the save)
    orders the next update after the copy, and what lands on disk is the state at the time of the save, not the
    state after the update that was enqueued right behind it."""
    from composed_mixture_of_experts_engine_b200.elastic.fault_monitor import AsyncCheckpointer, LocalNVMeAdapter
    from composed_mixture_of_experts_engine_b200.ops.optim import build_optimizer

    torch.manual_seed(21)
    net = torch.nn.Sequential(torch.nn.Linear(512, 1024, bias=False), torch.nn.Linear(1024, 512, bias=False)
                              ).cuda().to(torch.bfloat16)
    opt = build_optimizer(net, lr=1e-2, weight_decay=0.0)
    ck = AsyncCheckpointer(LocalNVMeAdapter(str(tmp_path / "l")), None, retention=4, workers=1)
    want = {}
    for step in (1, 2, 3):
        for p in net.parameters():
            p.main_grad.normal_()
        opt.step()
        want[step] = {k: v.detach().clone() for k, v in net.state_dict().items()}
        master = opt.groups[0].master.clone()
        ck.save(net, opt, step)
        if step == 1:
            first_allocs = ck._stager.allocations
        # the very next update is enqueued while the copy may still be running; its hook must order it behind
        for p in net.parameters():
            p.main_grad.normal_()
        opt.step()
        ck._q.join()
        got = ck.load_raw(step)
        for k, v in want[step].items():
            assert torch.equal(got["model"][k], v.cpu()), (step, k)
        assert torch.equal(got["optim"]["groups"]["dense"]["master"], master.cpu())
    assert first_allocs > 0 and ck._stager.allocations == first_allocs  # saves 2 and 3 reused the pinned set
    assert len(opt._pre_step_hooks) == 1 and ck.last_d2h_ms > 0.0
    # a weights-only save has no optimizer of its own to hook: `guard_with` names the one that updates the weights,
    # so this save too leaves the wait to that optimizer's next step, and the file holds the weights as they were
    want4 = {k: v.detach().clone() for k, v in net.state_dict().items()}
    ck.save(net, None, 4, guard_with=opt)
    assert ck._stager._pending is not None  # deferred, not waited for inside save()
    for p in net.parameters():
        p.main_grad.normal_()
    opt.step()
    assert ck._stager._pending is None
    ck._q.join()
    got = ck.load_raw(4)
    for k, v in want4.items():
        assert torch.equal(got["model"][k], v.cpu()), k
    ck.shutdown()


def test_trainer_loss_decreases_and_is_deterministic():
    from composed_mixture_of_experts_engine_b200.engine import Trainer
    from composed_mixture_of_experts_engine_b200.utils.config import MoEConfig

    def run():
        cfg = MoEConfig.from_dict({
            "model": dict(arch="moe_decoder", hidden_dim=256, num_layers=2, num_heads=4, num_experts=8, top_k=2,
                          ffn_dim=256, vocab_size=2048, sequence_length=256, dtype="bfloat16", aux_loss_coeff=0.01,
                          init_std=0.02),
            "training": dict(micro_batch_size=2, gradient_accumulation_steps=2, max_steps=100, warmup_steps=0,
                             learning_rate=1e-3, seed=5),
            "parallelism": dict(data_parallel=1, expert_parallel=1)})
        tr = Trainer(cfg)
        ids, tgt = tr.synthetic_batch(torch.Generator().manual_seed(0))
        return [float(tr.train_step(ids, tgt)) for _ in range(8)]

    a, b = run(), run()
    assert all(math.isfinite(v) for v in a) and a[-1] < a[0] - 0.2
    # same seed twice: bit-identical trajectories.  Every sum whose order could vary is taken in a fixed order (loss
    # rows, norm-weight gradients, the gradient norm that sets the clipping factor) or in integer fixed point (the
    # router's probability and z-loss sums), so a difference here means a race, not rounding.
    assert a == b


@pytest.mark.parametrize("nh,nkv", [(4, 4), (4, 2)])
def test_rope_attention_on_packed_projection_matches_fp32_restatement(nh, nkv):
    """The packed RoPE + attention op (in-place rotation, packed gradient) vs rope_reference + attention_reference
    in fp32 under plain autograd."""
    from composed_mixture_of_experts_engine_b200.ops import functional as OF
    from composed_mixture_of_experts_engine_b200.ops.attention import attention_reference

    torch.manual_seed(3)
    B, S, hd = 2, 256, 64
    heads = nh + 2 * nkv
    cos, sin = OF.rope_tables(S, hd, 10000.0, torch.device("cuda"))
    base = torch.randn(B, S, heads, hd, device="cuda")
    go = torch.randn(B, S, nh, hd, device="cuda")

    ref_in = base.clone().requires_grad_()
    t = OF.rope_reference(ref_in.reshape(B * S, heads, hd), cos, sin, S, nh + nkv).view(B, S, heads, hd)
    ref = attention_reference(t[:, :, :nh], t[:, :, nh: nh + nkv], t[:, :, nh + nkv:])
    ref.backward(go)

    x = base.to(torch.bfloat16).requires_grad_()
    out = OF.rope_causal_attention(x * 1.0, cos, sin, nh, nkv)  # x * 1.0: the op consumes its input buffer
    out.backward(go.to(torch.bfloat16))
    err = (out.float() - ref).norm() / ref.norm()
    gerr = (x.grad.float() - ref_in.grad).norm() / ref_in.grad.norm()
    assert err < 2e-2 and gerr < 3e-2, (float(err), float(gerr))
