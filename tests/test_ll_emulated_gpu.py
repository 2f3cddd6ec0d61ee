"""Low-latency dispatch / combine with emulated ranks on one GPU, against a pure-torch oracle.
Covers what tests/legacy/test_low_latency.py of the reference covers without RDMA: FP8 / BF16,
rounded and UE8M0 scales, receive hooks, repeated calls on the two buffer halves, CUDA-graph
replay, and the legacy front end on a one-rank group."""
import pytest
import torch

from conftest import make_routed_inputs

pytestmark = pytest.mark.gpu


def _cluster(R, T, H, E):
    import deepep_b200
    from deepep_b200.parallel.local_cluster import LocalCluster
    num_bytes = deepep_b200.Buffer.get_low_latency_rdma_size_hint(T, H, R, E)
    return LocalCluster(R, num_bytes=num_bytes, num_gpu_timeout_secs=5)


def _expected_rows(idxs, rank, le, EL):
    """(source rank, token, lane) of the rows local expert `le` of `rank` must hold, in order."""
    rows = []
    e = rank * EL + le
    for s, idx in enumerate(idxs):
        hit = (idx.cpu() == e)
        tok, lane = hit.nonzero(as_tuple=True)
        rows += [(s, int(t), int(k)) for t, k in zip(tok, lane)]
    return rows


@pytest.mark.parametrize('use_fp8,round_scale,use_ue8m0', [(True, False, False), (True, True, False), (True, True, True),
                                                           (False, False, False)])
def test_ll_dispatch_combine(use_fp8, round_scale, use_ue8m0):
    from deepep_b200.utils.math import per_token_cast_back, per_token_cast_to_fp8, unpack_ue8m0
    R, T, H, E, K = 4, 24, 1024, 32, 4
    EL = E // R
    cl = _cluster(R, T, H, E)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=11, device='cuda', masked_ratio=0.1)
    for call in range(3):   # both buffer halves, and a third call that reuses the first
        ios = cl.low_latency_dispatch(xs, idxs, T, E, use_fp8, round_scale, use_ue8m0, num_sms=8)
        torch.cuda.synchronize()
        cl.check_status()
        deq = []
        for r in range(R):
            io = ios[r]
            vals = torch.zeros((EL, R * T, H), dtype=torch.float32)
            for le in range(EL):
                rows = _expected_rows(idxs, r, le, EL)
                assert int(io.packed_recv_count[le].item()) == len(rows)
                if not rows:
                    continue
                src = torch.stack([xs[s][t] for s, t, _ in rows])
                info = torch.tensor([t | (k << 16) for _, t, k in rows], dtype=torch.int32)
                assert torch.equal(io.src_info[le, :len(rows)].cpu(), info)
                got = io.packed_recv_x[le, :len(rows)]
                if use_fp8:
                    q, sc = per_token_cast_to_fp8(src, round_scale=round_scale)
                    assert torch.equal(got.view(torch.uint8), q.view(torch.uint8))
                    sf = io.packed_recv_sf[le, :len(rows)]
                    assert io.packed_recv_sf.stride(1) == 1    # column-major in the last two dimensions
                    if use_ue8m0:
                        sf = unpack_ue8m0(sf.contiguous()).view(len(rows), -1)
                    assert torch.equal(sf.float(), sc)
                    vals[le, :len(rows)] = per_token_cast_back(q, sc).float().cpu()
                else:
                    assert torch.equal(got, src)
                    vals[le, :len(rows)] = src.float().cpu()
                # layout_range: (begin << 32 | count) per source rank
                begin = 0
                for s in range(R):
                    cnt = sum(1 for ss, _, _ in rows if ss == s)
                    assert int(io.layout_range[le, s].item()) == (begin << 32 | cnt)
                    begin += cnt
            deq.append(vals)
        ys = [(d * (1 + r)).bfloat16().cuda() for r, d in enumerate(deq)]
        cios = cl.low_latency_combine(ys, idxs, ws, ios, T, E, num_sms=8)
        torch.cuda.synchronize()
        cl.check_status()
        for r in range(R):
            ref = torch.zeros((xs[r].size(0), H), dtype=torch.float32)
            for t in range(xs[r].size(0)):
                for k in range(K):
                    e = int(idxs[r][t, k])
                    if e < 0:
                        continue
                    owner, le = e // EL, e % EL
                    rows = _expected_rows(idxs, owner, le, EL)
                    j = rows.index((r, t, k))
                    ref[t] = torch.addcmul(ref[t], ys[owner][le, j].float().cpu(), ws[r][t, k].cpu().float())
            got = cios[r].combined_x.float().cpu()
            assert torch.allclose(got, ref.bfloat16().float(), rtol=2e-2, atol=2e-2)
    cl.destroy()


def test_ll_combine_logfmt():
    """LogFMT-10 combine: groups below 1 in magnitude travel as 10-bit codes, others as bf16; hidden sizes with a
    partial pass of groups; checked against the torch restatement of the format and against the exact sum."""
    from deepep_b200.utils.math import calc_diff, logfmt_roundtrip
    for H in (1024, 1152, 7168):
        R, T, E, K = 4, 16, 16, 4
        EL = E // R
        cl = _cluster(R, T, H, E)
        xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=21, device='cuda', masked_ratio=0.1)
        for call in range(3):
            ios = cl.low_latency_dispatch(xs, idxs, T, E, False, num_sms=8)
            torch.cuda.synchronize()
            g = torch.Generator(device='cuda').manual_seed(100 + call)
            ys = []
            for r in range(R):
                y = torch.randn((EL, R * T, H), device='cuda', generator=g) * 0.1
                y[:, :, 128:256] *= 30.0            # a group that is too large to be cast
                y[:, :, 256:384] = 0.0              # an all-zero group
                y[:, :, 384:512] = 0.5              # a group with amin == amax
                y[:, ::3, 512:640] *= 1e-3          # rows with a different range
                y[:, :, 640] = 0.0                  # an exact zero inside a cast group
                ys.append(y.bfloat16())
            cios = cl.low_latency_combine(ys, idxs, ws, ios, T, E, num_sms=8, use_logfmt=True)
            torch.cuda.synchronize()
            cl.check_status()
            for r in range(R):
                Tr = xs[r].size(0)
                ref = torch.zeros((Tr, H), dtype=torch.float32, device='cuda')
                exact = torch.zeros_like(ref)
                for t in range(Tr):
                    for k in range(K):
                        e = int(idxs[r][t, k])
                        if e < 0:
                            continue
                        owner, le = e // EL, e % EL
                        j = _expected_rows(idxs, owner, le, EL).index((r, t, k))
                        row = ys[owner][le, j]
                        ref[t] += ws[r][t, k] * logfmt_roundtrip(row[None])[0]
                        exact[t] += ws[r][t, k] * row.float()
                got = cios[r].combined_x.float()
                assert calc_diff(got, ref) < 5e-6, (H, call, r, calc_diff(got, ref))
                assert calc_diff(got, exact) < 2e-4
                # groups that are not cast (too large, all zero, single value) differ by the final bf16 rounding only
                assert torch.allclose(got[:, 128:512], exact[:, 128:512], rtol=8e-3, atol=1e-6)
                assert not torch.equal(cios[r].combined_x, exact.bfloat16())   # the format was really used
            # the same buffers serve a plain bf16 combine afterwards
            cios = cl.low_latency_combine(ys, idxs, ws, ios, T, E, num_sms=8)
            torch.cuda.synchronize()
            cl.check_status()
        cl.destroy()


def test_ll_recv_hook_split():
    R, T, H, E, K = 2, 16, 512, 8, 2
    import deepep_b200
    C = deepep_b200._C
    cl = _cluster(R, T, H, E)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=12, device='cuda')
    ios = cl.low_latency_dispatch(xs, idxs, T, E, False, phases=C.LL_SEND, num_sms=4)
    cl.low_latency_dispatch(xs, idxs, T, E, False, phases=C.LL_RECV, ios=ios, num_sms=4)
    torch.cuda.synchronize()
    cl.check_status()
    full = cl.low_latency_dispatch(xs, idxs, T, E, False, num_sms=4)
    torch.cuda.synchronize()
    for a, b in zip(ios, full):
        assert torch.equal(a.packed_recv_count, b.packed_recv_count)
        assert torch.equal(a.layout_range, b.layout_range)
        for le in range(E // R):
            c = int(a.packed_recv_count[le].item())
            assert torch.equal(a.packed_recv_x[le, :c], b.packed_recv_x[le, :c])
    # the routing may come as int32 as well (EP_NUM_TOPK_IDX_BITS=32 builds of the reference): same result
    idxs32 = [i.int() for i in idxs]
    narrow = cl.low_latency_dispatch(xs, idxs32, T, E, False, num_sms=4)
    ys = [torch.randn((E // R, R * T, H), device='cuda').bfloat16() for _ in range(R)]
    out64 = [c.combined_x.clone() for c in cl.low_latency_combine(ys, idxs, ws, narrow, T, E, num_sms=4)]
    again = cl.low_latency_dispatch(xs, idxs32, T, E, False, num_sms=4)
    out32 = [c.combined_x.clone() for c in cl.low_latency_combine(ys, idxs32, ws, again, T, E, num_sms=4)]
    torch.cuda.synchronize()
    cl.check_status()
    for a, b, o64, o32 in zip(narrow, full, out64, out32):
        assert torch.equal(a.packed_recv_count, b.packed_recv_count) and torch.equal(a.layout_range, b.layout_range)
        assert torch.equal(o64, o32)
    cl.destroy()


def test_legacy_buffer_single_rank_and_graph():
    import deepep_b200
    from deepep_b200.parallel.local_cluster import SingleProcessGroup
    T, H, E, K = 32, 1024, 8, 2
    hint = max(deepep_b200.Buffer.get_low_latency_rdma_size_hint(T, H, 1, E),
               deepep_b200.Config().get_nvl_buffer_size_hint(H * 2, 1, 64, K))
    buf = deepep_b200.Buffer(SingleProcessGroup(), num_nvl_bytes=hint, num_rdma_bytes=hint, low_latency_mode=True,
                             num_gpu_timeout_secs=5)
    xs, idxs, ws = make_routed_inputs(1, T, H, E, K, seed=13, device='cuda')
    x, idx, w = xs[0], idxs[0], ws[0]
    # layout query + normal mode
    per_rank, _, per_expert, in_rank, _ = buf.get_dispatch_layout(idx, E)
    assert int(per_rank[0]) == T and int(per_expert.sum()) == T * K and bool(in_rank.all())
    per_rank32, _, per_expert32, _, _ = buf.get_dispatch_layout(idx.int(), E)
    assert torch.equal(per_rank32, per_rank) and torch.equal(per_expert32, per_expert)
    recv_x, recv_idx, recv_w, counts, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_tokens_per_rank=per_rank,
                                                               is_token_in_rank=in_rank, num_tokens_per_expert=per_expert)
    assert torch.equal(recv_x, x) and counts == per_expert.tolist()
    out, out_w, _ = buf.combine(recv_x, handle, topk_weights=recv_w)
    assert torch.equal(out, x)
    # low-latency mode, captured in a CUDA graph and replayed
    buf.clean_low_latency_buffer(T, H, E)
    static_x = x.clone()
    combined = torch.empty_like(x)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):   # warm-up outside the capture
            (rx, rsf), cnt, h, _, hook = buf.low_latency_dispatch(static_x, idx, T, E, return_recv_hook=True)
            hook()
            y = torch.zeros((E, T, H), dtype=torch.bfloat16, device='cuda')
            buf.low_latency_combine(y, idx, w, h, out=combined, return_recv_hook=True)[2]()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        (rx, rsf), cnt, h, _, hook = buf.low_latency_dispatch(static_x, idx, T, E, return_recv_hook=True)
        hook()
        deq = (rx.float() * rsf.repeat_interleave(128, dim=2)).bfloat16()
        buf.low_latency_combine(deq, idx, w, h, out=combined, return_recv_hook=True)[2]()
    for rep in range(3):
        static_x.copy_(x * (rep + 1))
        graph.replay()
        torch.cuda.synchronize()
        buf.check_status()
        ref = (x.float() * (rep + 1)).bfloat16().float()
        assert torch.allclose(combined.float(), ref, rtol=0.08, atol=0.08 * (rep + 1))
    buf.destroy()
