"""Single-GPU micro-benchmarks of the individual kernels (also the command that ncu captures wrap).

    python -m deepep_b200.utils.kernel_bench --op dispatch --tokens 8192 --iters 5
    python -m deepep_b200.utils.kernel_bench --op gemm --m 8192 --n 2304 --k 7168
    ncu --set full --clock-control none -k regex:dispatch_kernel -s 3 -c 1 -o prof \\
        python -m deepep_b200.utils.kernel_bench --op dispatch --tokens 8192 --iters 2 --warmup 3

Ops: ``dispatch`` (fused FP8 cast), ``dispatch_prequant``, ``dispatch_bf16``, ``combine``, ``gemm``,
``gemm_fp8_grouped``, ``ll`` (low-latency dispatch + combine), ``ops`` (router, SwiGLU, quantisation, transpose),
``ag_gemm`` / ``gemm_rs`` (fused tensor-parallel operators with emulated ranks), ``ht_emulated`` (dispatch + combine
with emulated ranks: all kernels of the multi-rank path). Times are CUDA-event means on one
rank (EP1: all traffic is local, so dispatch / combine show the SM-side cost of the kernels, not
NVLink).
"""
from __future__ import annotations

import argparse

import torch


def _timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--op', default='dispatch')
    ap.add_argument('--tokens', type=int, default=8192)
    ap.add_argument('--hidden', type=int, default=7168)
    ap.add_argument('--experts', type=int, default=256)
    ap.add_argument('--topk', type=int, default=8)
    ap.add_argument('--sms', type=int, default=24)
    ap.add_argument('--m', type=int, default=8192)
    ap.add_argument('--n', type=int, default=2304)
    ap.add_argument('--k', type=int, default=7168)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--ranks', type=int, default=2, help='ag_gemm / gemm_rs: emulated ranks')
    ap.add_argument('--baseline', action='store_true', help='gemm: also time torch.matmul on the same tensors')
    a = ap.parse_args()

    import deepep_b200
    from deepep_b200.parallel.local_cluster import SingleProcessGroup
    from deepep_b200.utils import gate
    from deepep_b200.utils.math import per_token_cast_to_fp8
    C = deepep_b200._C
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    T, H, E, K = a.tokens, a.hidden, a.experts, a.topk

    if a.op.startswith('dispatch') or a.op == 'combine':
        buf = deepep_b200.ElasticBuffer(SingleProcessGroup(), num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_gpu_timeout_secs=20)
        buf.runtime.enable_profiling(2)
        x = torch.randn((T, H), generator=g).bfloat16().cuda()
        idx, w = gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K)
        idx, w = idx.cuda(), w.cuda()
        xin, kw = x, dict(fused_fp8=True)
        if a.op == 'dispatch_prequant':
            xin, kw = per_token_cast_to_fp8(x), {}
        elif a.op == 'dispatch_bf16':
            kw = dict(fused_fp8=False)
        out = buf.dispatch(xin, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=a.sms, **kw)
        handle = out[3]
        y = torch.randn((handle.num_recv_tokens, H), device='cuda', dtype=torch.bfloat16)
        if a.op == 'combine':
            ms = _timeit(lambda: buf.combine(y, handle), a.iters, a.warmup)
        else:
            ms = _timeit(lambda: buf.dispatch(xin, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=a.sms, **kw), a.iters, a.warmup)
        t = buf.runtime.last_timings()
        print(f'{a.op}: {ms * 1e3:.1f} us per call (kernel {t[0 if a.op != "combine" else 2] * 1e3:.1f} us, '
              f'epilogue {t[1 if a.op != "combine" else 3] * 1e3:.1f} us), tokens {T}, hidden {H}, sms {a.sms}')
        buf.check_status()
        buf.destroy()
    elif a.op == 'gemm':
        x = torch.randn((a.m, a.k), generator=g).bfloat16().cuda()
        wt = torch.randn((a.n, a.k), generator=g).bfloat16().cuda()
        out = torch.empty((a.m, a.n), device='cuda', dtype=torch.bfloat16)
        ms = _timeit(lambda: C.gemm(x, wt, out=out), a.iters, a.warmup)
        print(f'gemm bf16 {a.m}x{a.n}x{a.k}: {ms * 1e3:.1f} us, {2 * a.m * a.n * a.k / ms / 1e9:.0f} TFLOP/s')
        if a.baseline:     # the library GEMM on the same tensors, as the yardstick only
            ms = _timeit(lambda: torch.matmul(x, wt.t(), out=out), a.iters, a.warmup)
            print(f'cuBLAS (torch.matmul) same tensors: {ms * 1e3:.1f} us, {2 * a.m * a.n * a.k / ms / 1e9:.0f} TFLOP/s')
    elif a.op == 'gemm_fp8_grouped':
        G, rows = 8, a.m // 8 // 128 * 128
        M = G * rows
        xq = torch.randn((M, a.k), generator=g).cuda().to(torch.float8_e4m3fn)
        sfa = torch.rand((M, a.k // 128), generator=g).cuda() + 0.5
        wq = torch.randn((G, a.n, a.k), generator=g).cuda().to(torch.float8_e4m3fn)
        sfb = torch.rand((G, a.n // 128, a.k // 128), generator=g).cuda() + 0.5
        ends = (torch.arange(1, G + 1, device='cuda') * rows).int()
        out = torch.empty((M, a.n), device='cuda', dtype=torch.bfloat16)
        ms = _timeit(lambda: C.gemm(xq, wq, sfa=sfa, sfb=sfb, group_end=ends, group_alignment=128, out=out), a.iters, a.warmup)
        print(f'gemm fp8 grouped {G}x{rows}x{a.n}x{a.k}: {ms * 1e3:.1f} us, {2 * M * a.n * a.k / ms / 1e9:.0f} TFLOP/s')
    elif a.op == 'gemm_fp8_grouped_mx':
        # the same problem with power-of-two scales: the tensor core applies them (kind::mxf8f6f4.block_scale)
        G, rows = 8, a.m // 8 // 128 * 128
        M = G * rows
        xq = torch.randn((M, a.k), generator=g).cuda().to(torch.float8_e4m3fn)
        sfa = torch.exp2(torch.randint(-3, 4, (M, a.k // 128), generator=g).float()).cuda()
        wq = torch.randn((G, a.n, a.k), generator=g).cuda().to(torch.float8_e4m3fn)
        sfb = torch.exp2(torch.randint(-3, 4, (G, a.n // 128, a.k // 128), generator=g).float()).cuda()
        ends = (torch.arange(1, G + 1, device='cuda') * rows).int()
        out = torch.empty((M, a.n), device='cuda', dtype=torch.bfloat16)
        ms = _timeit(lambda: C.gemm(xq, wq, sfa=sfa, sfb=sfb, group_end=ends, group_alignment=128, out=out, pow2_scales=True), a.iters, a.warmup)
        print(f'gemm fp8 grouped, hardware block scaling {G}x{rows}x{a.n}x{a.k}: {ms * 1e3:.1f} us, {2 * M * a.n * a.k / ms / 1e9:.0f} TFLOP/s')
    elif a.op == 'll':
        Tl = min(T, 128)
        hint = deepep_b200.Buffer.get_low_latency_rdma_size_hint(Tl, H, 1, E)
        ll = deepep_b200.Buffer(SingleProcessGroup(), num_rdma_bytes=hint, low_latency_mode=True, num_gpu_timeout_secs=20)
        x = torch.randn((Tl, H), generator=g).bfloat16().cuda()
        idx, w = gate.topk_from_scores(gate.get_balanced_scores(Tl, E, generator=g), K)
        idx, w = idx.cuda(), w.cuda()
        yy = torch.randn((E, Tl, H), device='cuda', dtype=torch.bfloat16)

        def step():
            _, _, h, _, _ = ll.low_latency_dispatch(x, idx, Tl, E)
            ll.low_latency_combine(yy, idx, w, h)
        ms = _timeit(step, a.iters, a.warmup)
        print(f'll dispatch+combine: {ms * 1e3:.1f} us, tokens {Tl}')
        ll.check_status()
        ll.destroy()
    elif a.op == 'll_graph':
        # the low-latency pair (FP8 dispatch + weighted BF16 combine) captured in a CUDA graph and replayed, with block
        # 0's phase stamps of both kernels; the stream is held back by a sleep kernel so that the replays are queued
        # when the clock starts (device time, not launch time)
        Tl = min(T, 128)
        hint = deepep_b200.Buffer.get_low_latency_rdma_size_hint(Tl, H, 1, E)
        ll = deepep_b200.Buffer(SingleProcessGroup(), num_rdma_bytes=hint, low_latency_mode=True, num_gpu_timeout_secs=10)
        x = torch.randn((Tl, H), generator=g).bfloat16().cuda()
        idx, w = gate.topk_from_scores(gate.get_balanced_scores(Tl, E, generator=g), K)
        idx, w = idx.cuda(), w.cuda()
        yy = torch.randn((E, Tl, H), device='cuda', dtype=torch.bfloat16)
        out = torch.empty_like(x)

        def pair():
            _, _, h, _, _ = ll.low_latency_dispatch(x, idx, Tl, E, use_fp8=True, num_sms=a.sms)
            ll.low_latency_combine(yy, idx, w, h, out=out, num_sms=a.sms)

        def dispatch_only():
            ll.low_latency_dispatch(x, idx, Tl, E, use_fp8=True, num_sms=a.sms)
        for name, fn in (('dispatch + combine', pair), ('dispatch', dispatch_only)):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            for _ in range(10):
                graph.replay()
            torch.cuda.synchronize()
            n = 100
            st = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
            en = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
            torch.cuda._sleep(int(4e7))
            for i in range(n):
                st[i].record()
                graph.replay()
                en[i].record()
            torch.cuda.synchronize()
            us = sorted(s0.elapsed_time(e0) * 1e3 for s0, e0 in zip(st, en))
            ph = [round(v / 1e3, 1) for v in ll.runtime.last_dispatch_phases()][:5]
            tl = [round(v / 1e3, 1) for v in ll.runtime.last_timeline()[8:]]
            print(f'll {name}, {a.sms} SMs, graph replay: p50 {us[n // 2]:.1f} us, min {us[0]:.1f} us; dispatch stamps {ph}, combine stamps {tl}')
        ll.check_status()
        ll.destroy()
    elif a.op == 'ht_emulated':
        # dispatch + combine with `--ranks` emulated ranks on this GPU: every kernel of the multi-rank path runs (count
        # exchange, epilogue, arrival-driven reduce), with local "peers"
        from deepep_b200.parallel.local_cluster import LocalCluster
        R = a.ranks
        cl = LocalCluster(R, num_max_tokens_per_rank=T, hidden=H, num_topk=K, use_fp8_dispatch=True, num_gpu_timeout_secs=20)
        xs = [torch.randn((T, H), generator=g).bfloat16().cuda() for _ in range(R)]
        routed = [gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K) for _ in range(R)]
        idxs, ws = [i.cuda() for i, _ in routed], [w.cuda() for _, w in routed]
        ys = {}

        def step():
            out = cl.dispatch([dict(x=xs[r], topk_idx=idxs[r], topk_weights=ws[r], num_experts=E, num_sms=a.sms, fused_fp8=True,
                                    zero_copy=True, do_cpu_sync=False) for r in range(R)])
            for r in range(R):
                if r not in ys:
                    ys[r] = torch.randn((out[r][0][0].size(0), H), device='cuda', dtype=torch.bfloat16)
            cl.combine([dict(x=ys[r], handle=out[r][3], topk_weights=out[r][2]) for r in range(R)])
        ms = _timeit(step, a.iters, a.warmup)
        print(f'dispatch + combine, {R} emulated ranks x {T} tokens, {a.sms} SMs per rank: {ms * 1e3:.1f} us per step')
        cl.check_status()
        cl.destroy()
    elif a.op == 'ops':
        # the small MoE operators: router top-k, SwiGLU (+ fused cast), SwiGLU backward, 1x128 quantisation, transpose
        rows, inter = a.m, a.k // 4 // 128 * 128
        logits = torch.randn((rows, E), generator=g).cuda()
        h1 = torch.randn((rows, 2 * inter), generator=g).bfloat16().cuda()
        da = torch.randn((rows, inter), generator=g).bfloat16().cuda()
        rw = torch.rand((rows,), generator=g).cuda()
        xr = torch.randn((rows, a.k), generator=g).bfloat16().cuda()
        for name, fn, nbytes in (
                ('router_topk', lambda: C.router_topk(logits, K), rows * E * 4),
                ('swiglu', lambda: C.swiglu(h1, rw), rows * inter * 6),
                ('swiglu + fp8 cast', lambda: C.swiglu(h1, rw, None, True), rows * inter * 5),
                ('swiglu_backward (+ activation, gate-weight gradient)', lambda: C.swiglu_backward(h1, da, rw, True), rows * inter * 12),
                ('quant_1x128', lambda: C.quant_1x128(xr), rows * a.k * 3),
                ('transpose_bf16', lambda: C.transpose_bf16(xr), rows * a.k * 4)):
            ms = _timeit(fn, a.iters, a.warmup)
            print(f'{name}: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s of algorithmic bytes (rows {rows})')
    elif a.op in ('ag_gemm', 'gemm_rs'):
        # the fused tensor-parallel operators with `--ranks` emulated ranks on this GPU (the device code of the real
        # multi-GPU run; the "peers" are local, so times show the kernel structure, not NVLink)
        from deepep_b200.parallel.local_cluster import VirtualRanks
        from deepep_b200.parallel.tp_fused import TensorParallelContext, fused_multi
        R = a.ranks
        Ml, Kd, N = a.m // R, a.k, a.n
        vr = VirtualRanks(R)
        ctxs = [TensorParallelContext(vr.groups[r], Ml, Kd, N, num_gpu_timeout_secs=10) for r in range(R)]
        vr.connect()
        gg = torch.Generator(device='cuda').manual_seed(1)
        if a.op == 'ag_gemm':
            xs = [torch.randn((Ml, Kd), device='cuda', generator=gg).bfloat16() for _ in range(R)]
            ws = [(torch.randn((N, Kd), device='cuda', generator=gg) * 0.05).bfloat16() for _ in range(R)]
            fn = lambda: fused_multi(ctxs, 'ag_gemm', xs, ws, num_comm_ctas=2, num_sms=a.sms)
            flops = 2.0 * R * Ml * N * Kd * R
        else:
            xs = [torch.randn((R * Ml, Kd // R), device='cuda', generator=gg).bfloat16() for _ in range(R)]
            ws = [(torch.randn((N, Kd // R), device='cuda', generator=gg) * 0.05).bfloat16() for _ in range(R)]
            fn = lambda: fused_multi(ctxs, 'gemm_rs', xs, ws, num_sms=a.sms)
            flops = 2.0 * R * Ml * N * (Kd // R) * R
        ms = _timeit(fn, a.iters, a.warmup)
        print(f'{a.op} with {R} emulated ranks ({a.sms} SMs each): {ms * 1e3:.1f} us, {flops / ms / 1e9:.0f} TFLOP/s over all ranks')
        for c in ctxs:
            c.check_status()
            c.destroy()
    else:
        raise SystemExit(f'unknown op {a.op}')


if __name__ == '__main__':
    main()
