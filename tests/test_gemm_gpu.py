"""tcgen05 GEMM family against plain PyTorch fp32 references: bf16, grouped bf16 (expert-major
row segments with alignment gaps), and e4m3 with 1x128 / 128x128 block scales."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(got, ref):
    return ((got.float() - ref.float()).norm() / ref.float().norm().clamp(min=1e-6)).item()


@pytest.mark.parametrize('pair', ['1', '0'])
@pytest.mark.parametrize('M,N,K', [(128, 128, 64), (256, 256, 512), (1000, 384, 1024), (1000, 512, 1024), (4096, 2304, 7168)])
def test_gemm_bf16(M, N, K, pair, monkeypatch):
    """`pair` selects the CTA-pair kernel (tcgen05 cta_group::2, 256-row tiles; used when N is a multiple of 256)
    or one CTA per 128-row tile."""
    import deepep_b200
    monkeypatch.setenv('EP_GEMM_CTA_PAIR', pair)
    g = torch.Generator(device='cuda').manual_seed(0)
    a = torch.randn((M, K), device='cuda', generator=g).bfloat16()
    b = (torch.randn((N, K), device='cuda', generator=g) * 0.05).bfloat16()
    out = deepep_b200._C.gemm(a, b)
    torch.cuda.synchronize()
    assert deepep_b200._C.gemm_check_status() == 0
    ref = a.float() @ b.float().t()
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize('pair', ['1', '0'])
@pytest.mark.parametrize('counts', [[200, 0, 130, 57], [100, 50, 300, 1], [128, 128, 700]])
def test_grouped_gemm_bf16_with_gaps(counts, pair, monkeypatch):
    import deepep_b200
    monkeypatch.setenv('EP_GEMM_CTA_PAIR', pair)
    G, N, K, align = len(counts), 256, 512, 128
    g = torch.Generator(device='cuda').manual_seed(1)
    ends, start = [], 0
    for c in counts:
        ends.append(start + c)
        start = -(-(start + c) // align) * align
    M = start
    a = torch.randn((M, K), device='cuda', generator=g).bfloat16()
    b = (torch.randn((G, N, K), device='cuda', generator=g) * 0.05).bfloat16()
    out = torch.full((M, N), 7.0, device='cuda', dtype=torch.bfloat16)
    deepep_b200._C.gemm(a, b, group_end=torch.tensor(ends, dtype=torch.int32, device='cuda'), group_alignment=align, out=out)
    torch.cuda.synchronize()
    assert deepep_b200._C.gemm_check_status() == 0
    start = 0
    for gi, c in enumerate(counts):
        ref = a[start:start + c].float() @ b[gi].float().t()
        if c:
            assert _rel_err(out[start:start + c], ref) < 1e-2
        nxt = -(-(start + c) // align) * align
        gap = out[start + c:nxt]
        assert bool(((gap == 7.0) | (gap == 0.0)).all())     # gaps hold zeros (rows of a computed tile) or stay untouched
        start = nxt


@pytest.mark.parametrize('pair', ['1', '0'])
@pytest.mark.parametrize('grouped', [False, True])
def test_gemm_fp8_block_scaled(grouped, pair, monkeypatch):
    """`pair`: 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2, kind::f8f6f4) or 128 x 128 tiles on lone CTAs."""
    import deepep_b200
    from deepep_b200.utils.math import per_token_cast_back, per_token_cast_to_fp8
    monkeypatch.setenv('EP_GEMM_FP8_PAIR', pair)
    G, M, N, K = (3 if grouped else 1), 384, 512, 1024
    g = torch.Generator(device='cuda').manual_seed(2)
    a = torch.randn((M, K), device='cuda', generator=g).bfloat16()
    aq, sfa = per_token_cast_to_fp8(a)
    w = torch.randn((G, N, K), device='cuda', generator=g) * 0.05
    # 128x128 block quantisation of the weights
    wb = w.view(G, N // 128, 128, K // 128, 128)
    amax = wb.abs().amax(dim=(2, 4)).clamp(1e-4)
    sfb = (amax / 448.0).contiguous()
    wq = (wb / sfb[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(G, N, K)
    w_deq = (wq.float().view(G, N // 128, 128, K // 128, 128) * sfb[:, :, None, :, None]).view(G, N, K)
    a_deq = per_token_cast_back(aq, sfa).float()
    if grouped:
        ends = torch.tensor([128, 256, 384], dtype=torch.int32, device='cuda')
        out = deepep_b200._C.gemm(aq, wq, sfa=sfa, sfb=sfb, group_end=ends, group_alignment=128)
        ref = torch.cat([a_deq[i * 128:(i + 1) * 128] @ w_deq[i].t() for i in range(3)])
    else:
        out = deepep_b200._C.gemm(aq, wq[0], sfa=sfa, sfb=sfb)
        ref = a_deq @ w_deq[0].t()
    torch.cuda.synchronize()
    assert deepep_b200._C.gemm_check_status() == 0
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize('pair', ['0', '1'])
@pytest.mark.parametrize('grouped', [False, True])
@pytest.mark.parametrize('M,N,K', [(384, 512, 1024), (256, 256, 7168)])
def test_gemm_fp8_hardware_block_scaling(grouped, M, N, K, pair, monkeypatch):
    """Power-of-two scales (UE8M0): the tensor core applies them itself and a tile accumulates over all of K in tensor
    memory. Scales differ per row, per 128-wide k-block and between the two 128-column halves of a 256-wide tile, so a
    scale factor that lands in the wrong lane, column or byte of tensor memory shows up as an error of a factor of two
    or more."""
    import deepep_b200
    from deepep_b200.utils.math import per_token_cast_back, per_token_cast_to_fp8
    monkeypatch.setenv('EP_GEMM_FP8_MX_PAIR', pair)     # '1': 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2)
    G = 3 if grouped else 1
    g = torch.Generator(device='cuda').manual_seed(5)
    # rows and k-blocks of very different magnitude -> very different scales
    a = torch.randn((M, K), device='cuda', generator=g) * torch.exp2(torch.randint(-6, 7, (M, 1), device='cuda', generator=g).float())
    a = (a.view(M, K // 128, 128) * torch.exp2(torch.randint(-3, 4, (M, K // 128, 1), device='cuda', generator=g).float())).view(M, K).bfloat16()
    aq, sfa = per_token_cast_to_fp8(a, round_scale=True)
    assert bool((torch.frexp(sfa)[0] == 0.5).all())          # exact powers of two
    w = torch.randn((G, N, K), device='cuda', generator=g) * 0.05
    wb = w.view(G, N // 128, 128, K // 128, 128) * torch.exp2(torch.randint(-4, 5, (G, N // 128, 1, K // 128, 1), device='cuda', generator=g).float())
    amax = wb.abs().amax(dim=(2, 4)).clamp(1e-4)
    sfb = torch.exp2(torch.ceil(torch.log2(amax / 448.0))).contiguous()
    wq = (wb / sfb[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(G, N, K)
    w_deq = (wq.float().view(G, N // 128, 128, K // 128, 128) * sfb[:, :, None, :, None]).view(G, N, K)
    a_deq = per_token_cast_back(aq, sfa).float()
    if grouped:
        rows = M // 128
        ends = torch.tensor([128 * min(rows, i + 1) for i in range(G)], dtype=torch.int32, device='cuda')
        out = deepep_b200._C.gemm(aq, wq, sfa=sfa, sfb=sfb, group_end=ends, group_alignment=128, pow2_scales=True)
        starts = [0] + ends.tolist()[:-1]
        ref = torch.cat([a_deq[s:e] @ w_deq[i].t() for i, (s, e) in enumerate(zip(starts, ends.tolist()))])
        n_rows = int(ends[-1].item())
        out, ref = out[:n_rows], ref[:n_rows]
    else:
        out = deepep_b200._C.gemm(aq, wq[0], sfa=sfa, sfb=sfb, pow2_scales=True)
        ref = a_deq @ w_deq[0].t()
    torch.cuda.synchronize()
    assert deepep_b200._C.gemm_check_status() == 0
    assert _rel_err(out, ref) < 1e-2
    # the software-scaled kernel on the same operands agrees
    soft = deepep_b200._C.gemm(aq, wq if grouped else wq[0], sfa=sfa, sfb=sfb, **(dict(group_end=ends, group_alignment=128) if grouped else {}))
    torch.cuda.synchronize()
    assert _rel_err(out, soft[:out.size(0)]) < 1e-2


def test_gemm_k_grouped_weight_gradients():
    """Groups along the contraction dimension: out[g] = A[:, rows of g] @ B[:, rows of g]^T for all groups in one launch,
    the ranges read from a device prefix array (aligned starts, zero padding between the groups, one empty group)."""
    import deepep_b200
    C = deepep_b200._C
    g = torch.Generator(device='cuda').manual_seed(11)
    M, N, align = 256, 512, 128
    counts = [200, 0, 129, 64]
    starts, ends, cursor = [], [], 0
    for c in counts:
        starts.append(cursor)
        ends.append(cursor + c)
        cursor = -(-(cursor + c) // align) * align
    K = max(cursor, align)
    a = torch.zeros((M, K), device='cuda', dtype=torch.bfloat16)
    b = torch.zeros((N, K), device='cuda', dtype=torch.bfloat16)
    for s, e in zip(starts, ends):
        a[:, s:e] = torch.randn((M, e - s), device='cuda', generator=g).bfloat16()
        b[:, s:e] = torch.randn((N, e - s), device='cuda', generator=g).bfloat16()
    out = C.gemm_k_grouped(a, b, torch.tensor(ends, device='cuda', dtype=torch.int32), len(counts), align)
    torch.cuda.synchronize()
    assert C.gemm_check_status() == 0
    for i, (s, e) in enumerate(zip(starts, ends)):
        ref = a[:, s:e].float() @ b[:, s:e].float().t()
        if e == s:
            assert out[i].float().abs().max().item() == 0
        else:
            assert ((out[i].float() - ref).norm() / ref.norm()).item() < 1e-2
