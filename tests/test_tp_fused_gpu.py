"""Fused all-gather -> GEMM and GEMM -> reduce-scatter with emulated ranks on one GPU, against
plain fp32 matmuls of the gathered / summed operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _contexts(R, Ml, K, N):
    from deepep_b200.parallel.local_cluster import VirtualRanks
    from deepep_b200.parallel.tp_fused import TensorParallelContext
    vr = VirtualRanks(R)
    ctxs = [TensorParallelContext(vr.groups[r], Ml, K, N, num_gpu_timeout_secs=5) for r in range(R)]
    vr.connect()
    return ctxs


def _rel(got, ref):
    return ((got.float() - ref).norm() / ref.norm()).item()


@pytest.mark.parametrize('pair', ['1', '0'])
@pytest.mark.parametrize('R', [1, 2, 4])
def test_all_gather_gemm(R, pair, monkeypatch):
    """`pair`: GEMM CTAs in clusters of two (tcgen05 cta_group::2) or one CTA per tile."""
    from deepep_b200.parallel.tp_fused import fused_multi
    monkeypatch.setenv('EP_TP_CTA_PAIR', pair)
    Ml, K, N = 256, 512, 512
    ctxs = _contexts(R, Ml, K, N)
    g = torch.Generator(device='cuda').manual_seed(5)
    for call in range(3):
        xs = [torch.randn((Ml, K), device='cuda', generator=g).bfloat16() for _ in range(R)]
        ws = [(torch.randn((N, K), device='cuda', generator=g) * 0.05).bfloat16() for _ in range(R)]
        outs = fused_multi(ctxs, 'ag_gemm', xs, ws, num_comm_ctas=2 if R > 1 else 0, num_sms=16)
        torch.cuda.synchronize()
        for c in ctxs:
            c.check_status()
        full = torch.cat(xs).float()
        for r in range(R):
            assert outs[r].shape == (R * Ml, N)
            assert _rel(outs[r], full @ ws[r].float().t()) < 1e-2
    for c in ctxs:
        c.destroy()


@pytest.mark.parametrize('fuse_own', ['1', '0'])
@pytest.mark.parametrize('pair', ['1', '0'])
@pytest.mark.parametrize('R', [1, 2, 4])
def test_gemm_reduce_scatter(R, pair, fuse_own, monkeypatch):
    """`fuse_own`: the epilogue of a rank's own rows adds the peers' partial tiles (the form used up to four ranks) or
    the own rows go through the partial buffer and a reduction pass follows the GEMM (more ranks)."""
    from deepep_b200.parallel.tp_fused import fused_multi
    monkeypatch.setenv('EP_TP_CTA_PAIR', pair)
    monkeypatch.setenv('EP_TP_RS_FUSE_OWN', fuse_own)
    Ml, Kl, N = 256, 256, 512
    ctxs = _contexts(R, Ml, 512, N)
    g = torch.Generator(device='cuda').manual_seed(6)
    for call in range(3):
        xs = [torch.randn((R * Ml, Kl), device='cuda', generator=g).bfloat16() for _ in range(R)]
        ws = [(torch.randn((N, Kl), device='cuda', generator=g) * 0.05).bfloat16() for _ in range(R)]
        outs = fused_multi(ctxs, 'gemm_rs', xs, ws, num_sms=12)
        torch.cuda.synchronize()
        for c in ctxs:
            c.check_status()
        partials = [xs[r].float() @ ws[r].float().t() for r in range(R)]
        total = torch.stack([p.bfloat16().float() for p in partials]).sum(dim=0)   # partials travel as bf16
        for r in range(R):
            assert outs[r].shape == (Ml, N)
            assert _rel(outs[r], total[r * Ml:(r + 1) * Ml]) < 1e-2
    for c in ctxs:
        c.destroy()
