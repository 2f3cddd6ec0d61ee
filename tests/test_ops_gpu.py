"""Small MoE operators against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('T,E,K', [(37, 16, 2), (300, 256, 8), (64, 2048, 32)])
def test_router_topk_softmax(T, E, K):
    import deepep_b200
    logits = torch.randn((T, E), device='cuda', generator=torch.Generator(device='cuda').manual_seed(0))
    idx, w = deepep_b200._C.router_topk(logits, K)
    vals, ref_idx = torch.topk(logits, K, dim=1, sorted=True)
    assert torch.equal(idx, ref_idx)
    assert torch.allclose(w, torch.softmax(vals, dim=1), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize('pow2,col_major', [(False, False), (True, False), (False, True)])
def test_quant_dequant_1x128(pow2, col_major):
    import deepep_b200
    from deepep_b200.utils.math import per_token_cast_back, per_token_cast_to_fp8
    x = torch.randn((333, 1024), device='cuda', generator=torch.Generator(device='cuda').manual_seed(1)).bfloat16()
    q, sf = deepep_b200._C.quant_1x128(x, pow2, col_major)
    rq, rsf = per_token_cast_to_fp8(x, round_scale=pow2)
    assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8)) and torch.equal(sf, rsf)
    if col_major:
        assert sf.stride(0) == 1
    back = deepep_b200._C.dequant_1x128(q, sf.contiguous())
    assert torch.equal(back, per_token_cast_back(rq, rsf))


def test_swiglu_forward_backward_and_fused_cast():
    import deepep_b200
    from deepep_b200.utils.math import per_token_cast_to_fp8
    C = deepep_b200._C
    g = torch.Generator(device='cuda').manual_seed(2)
    M, I = 200, 512
    x = torch.randn((M, 2 * I), device='cuda', generator=g).bfloat16()
    rw = torch.rand(M, device='cuda', generator=g)
    out, _ = C.swiglu(x, rw)
    xf = x.float().requires_grad_(True)
    ref = torch.nn.functional.silu(xf[:, :I]) * xf[:, I:] * rw[:, None]
    assert torch.allclose(out.float(), ref.detach(), rtol=2e-2, atol=2e-2)
    q, sf = C.swiglu(x, rw, None, True)
    rq, rsf = per_token_cast_to_fp8(out)
    assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8)) and torch.equal(sf, rsf)
    dout = torch.randn((M, I), device='cuda', generator=g).bfloat16()
    ref.backward(dout.float())
    dx = C.swiglu_backward(x, dout, rw)
    assert torch.allclose(dx.float(), xf.grad, rtol=3e-2, atol=3e-2)
    t = C.transpose_bf16(x)
    assert torch.equal(t, x.t().contiguous())


def test_ops_package_wrappers():
    """deepep_b200.ops: the typed entry points and their fp32 references agree."""
    from deepep_b200 import ops
    g = torch.Generator(device='cuda').manual_seed(3)
    a = torch.randn((300, 512), device='cuda', generator=g).bfloat16()
    b = (torch.randn((256, 512), device='cuda', generator=g) * 0.05).bfloat16()
    ref = ops.ref_gemm(a, b)
    assert ((ops.gemm(a, b).float() - ref).norm() / ref.norm()).item() < 1e-2
    # grouped, fp8 with block scales
    G, N, K = 3, 256, 512
    ends = torch.tensor([100, 300, 520], dtype=torch.int32, device='cuda')      # starts 0, 128, 384
    M = 640
    x = torch.randn((M, K), device='cuda', generator=g).bfloat16()
    w = (torch.randn((G, N, K), device='cuda', generator=g) * 0.05).bfloat16()
    out = ops.grouped_gemm(x, w, ends, 128)
    ref = ops.ref_grouped_gemm(x, w, ends, 128)
    for s0, e0 in ((0, 100), (128, 300), (384, 520)):
        assert ((out[s0:e0].float() - ref[s0:e0]).norm() / ref[s0:e0].norm()).item() < 1e-2
    xq, sfa = ops.quant_1x128(x)
    got8 = ops.gemm(xq, b.to(torch.float8_e4m3fn), sfa, torch.ones((2, 4), device='cuda'))
    ref8 = ops.ref_gemm(xq, b.to(torch.float8_e4m3fn), sfa, torch.ones((2, 4), device='cuda'))
    assert ((got8.float() - ref8).norm() / ref8.norm()).item() < 1e-2
    idx, wts = ops.router_topk(torch.randn((50, 64), device='cuda', generator=g), 4)
    assert idx.shape == (50, 4) and torch.allclose(wts.sum(dim=1), torch.ones(50, device='cuda'), atol=1e-5)
    y, _ = ops.swiglu(x)
    assert torch.allclose(y.float(), ops.ref_swiglu(x), rtol=2e-2, atol=2e-2)
    assert torch.equal(ops.transpose(x), x.t().contiguous())
    assert torch.equal(ops.dequant_1x128(xq, sfa), (xq.float() * sfa.repeat_interleave(128, dim=1)).bfloat16())


@pytest.mark.parametrize('rows,cols', [(64, 64), (200, 328), (130, 72), (1, 7), (512, 4096)])
def test_transpose_interior_edge_and_unaligned(rows, cols):
    """Interior tiles of aligned tensors take the 16-byte path, edge tiles and unaligned views the element-wise one."""
    import deepep_b200
    C = deepep_b200._C
    g = torch.Generator(device='cuda').manual_seed(rows * 1000 + cols)
    x = torch.randn((rows, cols), device='cuda', generator=g).bfloat16()
    assert torch.equal(C.transpose_bf16(x), x.t().contiguous())
    if cols > 8:     # a view whose rows start 2 bytes off a 16-byte boundary
        v = x[:, 1:]
        assert torch.equal(C.transpose_bf16(v), v.t().contiguous())
