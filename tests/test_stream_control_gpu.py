"""The option matrix of the reference's tests/elastic/test_ep.py:22-31 on the public single-process API: previous events,
asynchronous completion, allocation on the communication stream, handle copies, zero / one / two biases, and a
double run that must give identical bytes. One rank, so the expected values are closed-form."""
import itertools

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(T, H, E, K, seed):
    from deepep_b200.utils import gate
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, H), generator=g).bfloat16().cuda()
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K)
    idx[::7] = -1                                      # tokens that nobody takes
    return x, idx.cuda(), w.cuda(), g


@pytest.mark.parametrize('use_previous_event,async_finish,on_comm_stream,handle_copy',
                         list(itertools.product([False, True], repeat=4)))
def test_dispatch_combine_option_matrix(use_previous_event, async_finish, on_comm_stream, handle_copy):
    import deepep_b200
    from deepep_b200.parallel.local_cluster import SingleProcessGroup
    T, H, E, K = 96, 512, 8, 2
    buf = deepep_b200.ElasticBuffer(SingleProcessGroup(), num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_gpu_timeout_secs=5)
    x, idx, w, g = _inputs(T, H, E, K, 5)
    valid = (idx >= 0).any(dim=1)
    stats = torch.zeros(E, dtype=torch.int32, device='cuda')
    results = []
    for num_bias in (0, 1, 2):
        biases = [torch.randn((T, H), generator=g).bfloat16().cuda() for _ in range(num_bias)]
        # work that the communication has to wait for: the input is produced on a side stream
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            torch.cuda._sleep(int(2e6))
            x_late = x * 1
            event = deepep_b200.ElasticBuffer.capture() if use_previous_event else None
        if not use_previous_event:
            torch.cuda.current_stream().wait_stream(side)
        recv_x, recv_idx, recv_w, handle, ev = buf.dispatch(
            x_late, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=4, cumulative_local_expert_recv_stats=stats,
            previous_event=event, async_with_compute_stream=async_finish, allocate_on_comm_stream=on_comm_stream,
            do_handle_copy=handle_copy)
        if async_finish:
            ev.current_stream_wait()
        assert torch.equal(recv_x, x[valid]) and torch.equal(recv_idx, idx[valid]) and torch.equal(recv_w, w[valid])
        assert (handle.topk_idx.data_ptr() == idx.data_ptr()) == (not handle_copy)
        y = (recv_x.float() * 2).bfloat16()
        bias = None if num_bias == 0 else (biases[0] if num_bias == 1 else tuple(biases))
        before_epilogue = deepep_b200.ElasticBuffer.capture() if (use_previous_event and num_bias > 0) else None
        combined, combined_w, ev2 = buf.combine(y, handle, topk_weights=recv_w, bias=bias, previous_event_before_epilogue=before_epilogue,
                                                async_with_compute_stream=async_finish, allocate_on_comm_stream=on_comm_stream)
        if async_finish:
            ev2.current_stream_wait()
        ref = torch.zeros((T, H), dtype=torch.float32, device='cuda')
        ref[valid] = y.float()
        for b in biases:
            ref += b.float()
        assert torch.equal(combined, ref.bfloat16())
        assert torch.equal(combined_w, torch.where(idx >= 0, w, torch.zeros_like(w)))
        results.append(combined.clone())
        torch.cuda.synchronize()
        buf.check_status()
    # every dispatch of the loop counted its (token, expert) pairs once
    expect = torch.stack([(idx == e).sum() for e in range(E)]).int() * 3
    assert torch.equal(stats, expect)
    buf.destroy()


def test_double_run_is_bit_identical():
    """Same inputs twice through fresh buffers (several emulated ranks, FP8 and BF16): identical bytes everywhere."""
    from deepep_b200.parallel.local_cluster import LocalCluster
    from deepep_b200.utils.math import hash_tensors
    from conftest import make_routed_inputs
    R, T, H, E, K = 4, 80, 512, 16, 4
    hashes = []
    for run in range(2):
        cl = LocalCluster(R, num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_gpu_timeout_secs=5)
        xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=9, device='cuda', masked_ratio=0.1)
        h = []
        for fused_fp8 in (False, True):
            out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=3, fused_fp8=fused_fp8,
                                    do_expand=True, expert_alignment=16, do_zero_padding=True) for r in range(R)])
            torch.cuda.synchronize()
            for r in range(R):
                rx = out[r][0]
                parts = list(rx) if isinstance(rx, tuple) else [rx]
                h.append(hash_tensors(*[p.view(torch.uint8) if p.dtype == torch.float8_e4m3fn else p for p in parts], out[r][2],
                                      out[r][3].recv_src_metadata, out[r][3].psum_num_recv_tokens_per_expert))
        ys = [torch.randn(out[r][0][0].shape, generator=torch.Generator().manual_seed(r)).bfloat16().cuda() for r in range(R)]
        comb = cl.combine([dict(x=ys[r], handle=out[r][3]) for r in range(R)])
        torch.cuda.synchronize()
        cl.check_status()
        h += [hash_tensors(comb[r][0]) for r in range(R)]
        hashes.append(h)
        cl.destroy()
    assert hashes[0] == hashes[1]
