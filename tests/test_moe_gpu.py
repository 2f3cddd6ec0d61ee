"""Fused MoE layer forward + backward (bf16 and FP8 forward) with emulated ranks, against a dense
fp32 PyTorch reference with autograd; plus the single-rank nn.Module path."""
import pytest
import torch

from conftest import make_routed_inputs

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-6)).item()


@pytest.mark.parametrize('use_fp8', [False, True, 'pow2'])
def test_moe_forward_backward_emulated(use_fp8):
    pow2 = use_fp8 == 'pow2'       # power-of-two scales: the expert GEMMs use the block-scaled tensor-core instruction
    use_fp8 = bool(use_fp8)
    from deepep_b200.models.moe import ExpertWeights, MoEConfig, moe_backward, moe_forward, reference_moe
    from deepep_b200.parallel.local_cluster import LocalCluster
    R, T, H, I, E, K = 2, 96, 256, 256, 8, 2
    EL = E // R
    # poison the allocator's free blocks: padding rows and their scales must not leak stale memory into the result
    junk = torch.full((64 << 20,), float('nan'), device='cuda')
    del junk
    cfg = MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, use_fp8=use_fp8, pow2_scales=pow2, num_sms=4)
    cl = LocalCluster(R, num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_gpu_timeout_secs=5)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=21, device='cuda', vary_tokens=True)
    g = torch.Generator(device='cuda').manual_seed(3)
    w13_all = (torch.randn((E, 2 * I, H), device='cuda', generator=g) * 0.05).bfloat16()
    w2_all = (torch.randn((E, H, I), device='cuda', generator=g) * 0.05).bfloat16()
    weights = [ExpertWeights(w13_all[r * EL:(r + 1) * EL], w2_all[r * EL:(r + 1) * EL], use_fp8, pow2) for r in range(R)]

    ys, ctxs = moe_forward(cl, weights, xs, idxs, ws, cfg)
    torch.cuda.synchronize()
    cl.check_status()
    # reference with autograd
    xr = [x.float().requires_grad_(True) for x in xs]
    wr = [w.float().requires_grad_(True) for w in ws]
    w13r, w2r = w13_all.float().requires_grad_(True), w2_all.float().requires_grad_(True)
    refs = reference_moe(xr, idxs, wr, w13r, w2r)
    tol = (0.1 if pow2 else 0.08) if use_fp8 else 0.03
    for r in range(R):
        assert _rel(ys[r], refs[r]) < tol

    dys = [torch.randn(y.shape, device='cuda', generator=g).bfloat16() for y in ys]
    dxs, dws, dW13s, dW2s = moe_backward(cl, weights, ctxs, dys, cfg)
    torch.cuda.synchronize()
    cl.check_status()
    torch.autograd.backward(refs, [d.float() for d in dys])
    for r in range(R):
        assert _rel(dxs[r], xr[r].grad) < tol + 0.02
        valid = idxs[r] >= 0
        assert _rel(torch.where(valid, dws[r], torch.zeros_like(dws[r])), torch.where(valid, wr[r].grad, torch.zeros_like(wr[r].grad))) < tol + 0.03
        assert _rel(dW13s[r], w13r.grad[r * EL:(r + 1) * EL]) < tol + 0.03
        assert _rel(dW2s[r], w2r.grad[r * EL:(r + 1) * EL]) < tol + 0.03
    cl.destroy()


def test_moe_module_single_rank_trains():
    import deepep_b200
    from deepep_b200.models.moe import FusedMoE, MoEConfig
    from deepep_b200.parallel.local_cluster import SingleProcessGroup
    T, H, I, E, K = 128, 256, 128, 4, 2
    buf = deepep_b200.ElasticBuffer(SingleProcessGroup(), num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_gpu_timeout_secs=5)
    layer = FusedMoE(buf, MoEConfig(hidden=H, intermediate=I, num_experts=E, num_topk=K, num_sms=4))
    x = torch.randn((T, H), device='cuda', generator=torch.Generator(device='cuda').manual_seed(4)).bfloat16().requires_grad_(True)
    y = layer(x)
    loss = (y.float() ** 2).mean()
    loss.backward()
    torch.cuda.synchronize()
    buf.check_status()
    assert y.shape == (T, H) and torch.isfinite(y.float()).all()
    for p in (x, layer.router, layer.w13, layer.w2):
        assert p.grad is not None and torch.isfinite(p.grad.float()).all() and p.grad.float().abs().sum() > 0
    buf.destroy()
