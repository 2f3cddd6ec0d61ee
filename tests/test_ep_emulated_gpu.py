"""High-throughput dispatch / combine on ONE GPU with emulated ranks, checked bitwise against the
pure-torch oracle. Mirrors the workload matrix of tests/elastic/test_ep.py of the reference
(plain, expanded, cached, FP8, bias, no-CPU-sync) at shapes small enough for one device."""
import pytest
import torch

from conftest import make_routed_inputs

pytestmark = pytest.mark.gpu


def _cluster(num_ranks, num_max_tokens, hidden, num_topk, fuse_reduce=None, **kw):
    # fuse_reduce: 0 reduce kernel after the send kernel, 1 arrival-driven reduce kernel beside it
    from deepep_b200.parallel.local_cluster import LocalCluster
    cl = LocalCluster(num_ranks, num_max_tokens_per_rank=num_max_tokens, hidden=hidden, num_topk=num_topk,
                      num_gpu_timeout_secs=5, num_cpu_timeout_secs=20, **kw)
    if fuse_reduce is not None:
        for b in cl.buffers:
            b.fuse_combine_reduce = fuse_reduce
    return cl


def _oracle(xs, idxs, ws, num_experts, num_max_tokens, sfs=None):
    from deepep_b200.utils import refs
    cpu = lambda ts: [t.cpu() for t in ts]
    raw = [x.view(torch.uint8).cpu() if x.dtype == torch.float8_e4m3fn else x.cpu() for x in xs]
    return [refs.dispatch_local(raw, cpu(idxs), cpu(ws), r, num_experts, num_max_tokens,
                                sfs=None if sfs is None else cpu(sfs)) for r in range(len(xs))]


def _as_bytes(t):
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


@pytest.mark.parametrize('num_ranks,num_tokens,hidden,num_experts,num_topk,num_sms', [
    (1, 33, 256, 8, 2, 4),
    (2, 64, 512, 16, 4, 3),
    (2, 40, 384, 8, 2, 2),      # 768-byte rows: the reduce epilogue cannot cut them into 512-byte chunks
    (4, 96, 1024, 32, 6, 4),
    (8, 128, 7168, 256, 8, 6),
    (8, 96, 7168, 256, 8, 18),  # eight ranks on many SMs: the number of send warps is capped below what shared memory allows
])
@pytest.mark.parametrize('fuse_reduce', [0, 1])
def test_dispatch_combine_bf16(num_ranks, num_tokens, hidden, num_experts, num_topk, num_sms, fuse_reduce):
    from deepep_b200.utils import refs
    T_max = num_tokens
    cl = _cluster(num_ranks, T_max, hidden, num_topk, fuse_reduce=fuse_reduce)
    xs, idxs, ws = make_routed_inputs(num_ranks, num_tokens, hidden, num_experts, num_topk, seed=1, device='cuda',
                                      masked_ratio=0.05)
    for idx in idxs:
        idx[::9] = -1       # whole tokens that nobody takes: they must come back as zeros (+ bias)
    stats = [torch.zeros(num_experts // num_ranks, dtype=torch.int32, device='cuda') for _ in range(num_ranks)]
    out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=num_experts, num_sms=num_sms,
                            cumulative_local_expert_recv_stats=stats[r]) for r in range(num_ranks)])
    torch.cuda.synchronize()
    cl.check_status()
    exp = _oracle(xs, idxs, ws, num_experts, T_max)
    for r in range(num_ranks):
        recv_x, recv_idx, recv_w, handle, _ = out[r]
        e = exp[r]
        assert handle.num_recv_tokens == e['recv_x'].size(0)
        assert torch.equal(recv_x.cpu(), e['recv_x'])
        assert torch.equal(recv_idx.cpu(), e['recv_topk_idx'])
        assert torch.equal(recv_w.cpu(), e['recv_topk_weights'])
        assert torch.equal(handle.recv_src_metadata[:, 0].cpu(), e['recv_src_token_idx'])
        assert torch.equal(handle.psum_num_recv_tokens_per_scaleup_rank.cpu(),
                           torch.cumsum(e['num_recv_tokens_per_rank'], 0).int())
        per_expert = torch.stack([(e['recv_topk_idx'] == le).sum() for le in range(num_experts // num_ranks)]).int()
        assert torch.equal(handle.num_unaligned_recv_tokens_per_expert.cpu(), per_expert)
        assert handle.num_recv_tokens_per_expert_list == per_expert.tolist()
        assert torch.equal(stats[r].cpu(), per_expert)

    # combine: every rank returns what it received, scaled per holder so that the order matters
    ys = [(out[r][0].float() * (1 + 0.25 * r)).bfloat16() for r in range(num_ranks)]
    g = torch.Generator().manual_seed(7)
    bias = [torch.randn((xs[r].size(0), hidden), generator=g).bfloat16().cuda() for r in range(num_ranks)]
    comb = cl.combine([dict(x=ys[r], handle=out[r][3], topk_weights=out[r][2], bias=bias[r]) for r in range(num_ranks)])
    torch.cuda.synchronize()
    cl.check_status()
    srcs = [out[r][3].recv_src_metadata[:, 0].cpu() for r in range(num_ranks)]
    for r in range(num_ranks):
        combined_x, combined_w, _ = comb[r]
        ref = refs.combine_local([y.cpu() for y in ys], srcs, r, xs[r].size(0), T_max, [bias[r].cpu()])
        assert torch.equal(combined_x.cpu(), ref)
        valid = idxs[r] >= 0
        assert torch.equal(torch.where(valid, combined_w, torch.zeros_like(combined_w)).cpu(),
                           torch.where(valid, ws[r], torch.zeros_like(ws[r])).cpu())
    # without a bias (a single rank then writes the result from the send kernel, tokens nobody took are zeroed there)
    comb = cl.combine([dict(x=ys[r], handle=out[r][3], topk_weights=out[r][2]) for r in range(num_ranks)])
    torch.cuda.synchronize()
    cl.check_status()
    for r in range(num_ranks):
        ref = refs.combine_local([y.cpu() for y in ys], srcs, r, xs[r].size(0), T_max)
        assert torch.equal(comb[r][0].cpu(), ref)
        valid = idxs[r] >= 0
        assert torch.equal(comb[r][1].cpu(), torch.where(valid, ws[r], torch.zeros_like(ws[r])).cpu())
    cl.destroy()


@pytest.mark.parametrize('fused', [False, True])
@pytest.mark.parametrize('col_major', [False, True])
def test_dispatch_fp8(fused, col_major):
    from deepep_b200.utils.math import per_token_cast_to_fp8
    R, T, H, E, K = 4, 80, 1024, 32, 4
    cl = _cluster(R, T, H, K, use_fp8_dispatch=True)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=2, device='cuda')
    q = [per_token_cast_to_fp8(x) for x in xs]
    if fused:
        kw = [dict(x=xs[r], fused_fp8=True) for r in range(R)]
    else:
        kw = [dict(x=(q[r][0], q[r][1])) for r in range(R)]
    out = cl.dispatch([dict(topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=4,
                            use_tma_aligned_col_major_sf=col_major, **kw[r]) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    exp = _oracle([a for a, _ in q], idxs, ws, E, T, sfs=[b for _, b in q])
    for r in range(R):
        (recv_x, recv_sf), recv_idx, recv_w, handle, _ = out[r]
        assert recv_x.dtype == torch.float8_e4m3fn
        assert torch.equal(recv_x.view(torch.uint8).cpu(), exp[r]['recv_x'])
        assert torch.equal(recv_sf.cpu(), exp[r]['recv_sf'])
        if col_major:
            assert recv_sf.stride(0) == 1 and recv_sf.stride(1) % 4 == 0
        assert torch.equal(recv_idx.cpu(), exp[r]['recv_topk_idx'])
    cl.destroy()


@pytest.mark.parametrize('alignment,zero_padding', [(1, False), (16, True)])
@pytest.mark.parametrize('fuse_reduce', [0, 1])
def test_dispatch_expand_and_combine(alignment, zero_padding, fuse_reduce):
    from deepep_b200.utils import refs
    R, T, H, E, K = 4, 72, 512, 16, 3
    cl = _cluster(R, T, H, K, fuse_reduce=fuse_reduce)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=3, device='cuda', masked_ratio=0.1)
    out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=3, do_expand=True,
                            expert_alignment=alignment, do_zero_padding=zero_padding) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    exp = _oracle(xs, idxs, ws, E, T)
    EL = E // R
    for r in range(R):
        recv_x, recv_idx, recv_w, handle, _ = out[r]
        assert recv_idx is None
        ex = refs.expand_local(exp[r], EL, alignment)
        assert handle.num_expanded_tokens == ex['num_rows'] == recv_x.size(0)
        psum = handle.psum_num_recv_tokens_per_expert.cpu()
        for le in range(EL):
            s, c = int(ex['starts'][le]), int(ex['counts'][le])
            assert int(psum[le]) == s + c
            rows = ex['row_of'][le]
            assert torch.equal(recv_x[s:s + c].cpu(), exp[r]['recv_x'][rows])
            lanes = (exp[r]['recv_topk_idx'][rows] == le).float().argmax(dim=1)
            assert torch.equal(recv_w[s:s + c].cpu(), exp[r]['recv_topk_weights'][rows, lanes])
            if zero_padding:
                end = -(-(s + c) // alignment) * alignment
                assert recv_x[s + c:end].float().abs().sum().item() == 0
        assert torch.equal(handle.recv_src_metadata[:, 2:].cpu().long(), ex['lane_rows'])

    # expanded combine: one row per (token, expert); each rank pre-reduces its rows
    ys = [torch.randn(out[r][0].shape, generator=torch.Generator().manual_seed(10 + r)).bfloat16().cuda() for r in range(R)]
    comb = cl.combine([dict(x=ys[r], handle=out[r][3]) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    partial, srcs = [], []
    for r in range(R):
        lane_rows = out[r][3].recv_src_metadata[:, 2:].cpu().long()
        acc = torch.zeros((lane_rows.size(0), H), dtype=torch.float32)
        y = ys[r].cpu().float()
        for k in range(K):
            ok = lane_rows[:, k] >= 0
            acc[ok] += y[lane_rows[ok, k]]
        partial.append(acc.bfloat16())
        srcs.append(out[r][3].recv_src_metadata[:, 0].cpu())
    for r in range(R):
        ref = refs.combine_local(partial, srcs, r, xs[r].size(0), T)
        assert torch.equal(comb[r][0].cpu(), ref)
    cl.destroy()


@pytest.mark.parametrize('fuse_reduce', [0, 1])
def test_combine_topk_layout_single_rounding(fuse_reduce):
    """allow_multiple_reduction=False: every expert row travels on its own and the source rank sums them in fp32 in
    ascending top-k order with one rounding."""
    R, T, H, E, K = 4, 40, 512, 16, 4
    EL = E // R
    cl = _cluster(R, T, H, K, fuse_reduce=fuse_reduce, allow_multiple_reduction=False)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=5, device='cuda', masked_ratio=0.1)
    out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=3, do_expand=True)
                       for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    for call in range(2):
        ys = [torch.randn(out[r][0].shape, generator=torch.Generator().manual_seed(20 + 10 * call + r)).bfloat16().cuda()
              for r in range(R)]
        comb = cl.combine([dict(x=ys[r], handle=out[r][3]) for r in range(R)])
        torch.cuda.synchronize()
        cl.check_status()
        for r in range(R):
            rows = out[r][3].dst_expanded_row_idx.cpu()
            ref = torch.zeros((xs[r].size(0), H), dtype=torch.float32)
            for k in range(K):
                e = idxs[r][:, k].cpu()
                for t in range(xs[r].size(0)):
                    if e[t] >= 0:
                        ref[t] += ys[int(e[t]) // EL][int(rows[t, k])].cpu().float()
            assert torch.equal(comb[r][0].cpu(), ref.bfloat16())
    cl.destroy()


def test_cached_dispatch_no_cpu_sync_zero_copy():
    R, T, H, E, K = 4, 64, 512, 32, 4
    cl = _cluster(R, T, H, K)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=4, device='cuda')
    first = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=4) for r in range(R)])
    exp = _oracle(xs, idxs, ws, E, T)
    # cached replay with new payload, zero-copy output
    xs2 = [(x.float() * 2 + 1).bfloat16() for x in xs]
    exp2 = _oracle(xs2, idxs, ws, E, T)
    second = cl.dispatch([dict(x=xs2[r], handle=first[r][3], topk_weights=ws[r], zero_copy=True) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    for r in range(R):
        assert torch.equal(second[r][0].cpu(), exp2[r]['recv_x'])
        assert torch.equal(second[r][1].cpu(), exp2[r]['recv_topk_idx'])
    # no CPU sync: worst-case shapes, true count on the device
    third = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=4, do_cpu_sync=False)
                         for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    for r in range(R):
        recv_x, _, _, handle, _ = third[r]
        n = int(handle.psum_num_recv_tokens_per_scaleup_rank[-1].item())
        assert recv_x.size(0) == R * T and n == exp[r]['recv_x'].size(0)
        assert torch.equal(recv_x[:n].cpu(), exp[r]['recv_x'])
    # ... and the combine takes the worst-case shaped tensor as it is (the true row count is read on the device)
    from deepep_b200.utils import refs
    comb = cl.combine([dict(x=third[r][0], handle=third[r][3]) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    ns = [int(third[r][3].psum_num_recv_tokens_per_scaleup_rank[-1].item()) for r in range(R)]
    srcs = [third[r][3].recv_src_metadata[:ns[r], 0].cpu() for r in range(R)]
    for r in range(R):
        ref = refs.combine_local([third[q][0][:ns[q]].cpu() for q in range(R)], srcs, r, xs[r].size(0), T)
        assert torch.equal(comb[r][0].cpu(), ref)
    cl.destroy()


def test_zero_copy_views_of_the_receive_region():
    """zero_copy: payload and row-major scales are strided views of the records where they landed."""
    from deepep_b200.utils.math import per_token_cast_to_fp8
    R, T, H, E, K = 4, 80, 1024, 32, 4
    cl = _cluster(R, T, H, K, use_fp8_dispatch=True)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=12, device='cuda')
    q = [per_token_cast_to_fp8(x) for x in xs]
    out = cl.dispatch([dict(x=xs[r], fused_fp8=True, topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=4,
                            zero_copy=True) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    exp = _oracle([a for a, _ in q], idxs, ws, E, T, sfs=[b for _, b in q])
    for r in range(R):
        (recv_x, recv_sf), recv_idx, recv_w, handle, _ = out[r]
        assert recv_x.stride(0) > H and recv_x.stride(0) % 128 == 0 and recv_x.stride(1) == 1      # rows sit a record apart
        assert recv_sf.stride(0) * 4 == recv_x.stride(0) and recv_sf.stride(1) == 1
        assert torch.equal(recv_x.view(torch.uint8).cpu(), exp[r]['recv_x'])
        assert torch.equal(recv_sf.cpu(), exp[r]['recv_sf'])
        assert torch.equal(recv_idx.cpu(), exp[r]['recv_topk_idx'])
        assert torch.equal(recv_w.cpu(), exp[r]['recv_topk_weights'])
    cl.destroy()


def test_int32_topk_idx():
    """Routing indices may be int32 (EP_NUM_TOPK_IDX_BITS=32 of the reference): same rows, int32 local ids back."""
    from deepep_b200.utils import refs
    R, T, H, E, K = 4, 48, 512, 16, 4
    cl = _cluster(R, T, H, K)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=13, device='cuda', masked_ratio=0.1)
    out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r].int(), topk_weights=ws[r], num_experts=E, num_sms=3) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    exp = _oracle(xs, idxs, ws, E, T)
    for r in range(R):
        recv_x, recv_idx, recv_w, handle, _ = out[r]
        assert recv_idx.dtype == torch.int32 and handle.topk_idx.dtype == torch.int32
        assert torch.equal(recv_x.cpu(), exp[r]['recv_x'])
        assert torch.equal(recv_idx.cpu().long(), exp[r]['recv_topk_idx'])
        counts = handle.num_tokens_per_rank_matrix.cpu()
        assert int(counts[:, r].sum()) == recv_x.size(0)
    comb = cl.combine([dict(x=out[r][0], handle=out[r][3]) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    srcs = [out[r][3].recv_src_metadata[:, 0].cpu() for r in range(R)]
    for r in range(R):
        ref = refs.combine_local([out[q][0].cpu() for q in range(R)], srcs, r, xs[r].size(0), T)
        assert torch.equal(comb[r][0].cpu(), ref)
    cl.destroy()


def test_num_worst_tokens_fills_the_tail():
    """Without CPU sync and with ``num_worst_tokens``: outputs have exactly that many rows; routing rows past the
    received count hold -1 / 0 even when the memory was poisoned before."""
    R, T, H, E, K = 4, 32, 256, 16, 2
    cl = _cluster(R, T, H, K)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=14, device='cuda')
    worst = 100
    out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=2, do_cpu_sync=False,
                            num_worst_tokens=worst) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    exp = _oracle(xs, idxs, ws, E, T)
    for r in range(R):
        recv_x, recv_idx, recv_w, handle, _ = out[r]
        n = exp[r]['recv_x'].size(0)
        assert recv_x.size(0) == worst and recv_idx.size(0) == worst and n <= worst
        assert torch.equal(recv_x[:n].cpu(), exp[r]['recv_x'])
        assert torch.equal(recv_idx[:n].cpu(), exp[r]['recv_topk_idx'])
        assert (recv_idx[n:] == -1).all() and (recv_w[n:] == 0).all()
        assert (handle.recv_src_metadata[n:] == -1).all()
    cl.destroy()


@pytest.mark.parametrize('allow_multiple_reduction', [True, False])
@pytest.mark.parametrize('fuse_reduce', [0, 1])
def test_weighted_combine(allow_multiple_reduction, fuse_reduce):
    """weighted=True on the expanded layout: combined_x[t] = sum_k w[t, k] * y_k (fp32 accumulation)."""
    R, T, H, E, K = 4, 40, 512, 16, 4
    EL = E // R
    cl = _cluster(R, T, H, K, fuse_reduce=fuse_reduce, allow_multiple_reduction=allow_multiple_reduction)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=15, device='cuda', masked_ratio=0.1)
    out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=3, do_expand=True)
                       for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    ys = [torch.randn(out[r][0].shape, generator=torch.Generator().manual_seed(30 + r)).bfloat16().cuda() for r in range(R)]
    comb = cl.combine([dict(x=ys[r], handle=out[r][3], topk_weights=out[r][2], weighted=True) for r in range(R)])
    torch.cuda.synchronize()
    cl.check_status()
    for r in range(R):
        rows = out[r][3].dst_expanded_row_idx.cpu()
        ref = torch.zeros((xs[r].size(0), H), dtype=torch.float32)
        for k in range(K):
            e = idxs[r][:, k].cpu()
            for t in range(xs[r].size(0)):
                if e[t] >= 0:
                    ref[t] += float(ws[r][t, k]) * ys[int(e[t]) // EL][int(rows[t, k])].cpu().float()
        got = comb[r][0].cpu().float()
        assert torch.allclose(got, ref, rtol=2e-2, atol=2e-2)
        assert (got - ref).abs().max().item() < 0.1
    cl.destroy()


def test_barrier_and_repeat():
    cl = _cluster(4, 16, 256, 2)
    for _ in range(5):
        cl.barrier(with_cpu_sync=True)
    cl.destroy()
