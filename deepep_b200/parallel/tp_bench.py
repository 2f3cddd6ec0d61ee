"""Multi-GPU micro-benchmark of the fused tensor-parallel operators against NCCL + cuBLAS.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29531 \\
        -m deepep_b200.parallel.tp_bench --tokens 8192 --hidden 7168 --ffn 18432 --comm-ctas 8,16,32

Every figure is a CUDA-event mean on the launching stream, ranks released together by a GPU sleep and an
all-reduce before each call, maximum over ranks. Prints relative errors against the baselines first.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--tokens', type=int, default=8192)
    ap.add_argument('--hidden', type=int, default=7168)
    ap.add_argument('--ffn', type=int, default=18432)
    ap.add_argument('--comm-ctas', default='8,16,24')
    ap.add_argument('--iters', type=int, default=10)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1)), int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    dist.init_process_group('nccl', device_id=dev)
    group = dist.group.WORLD
    from deepep_b200.parallel.tp_fused import TensorParallelContext, nccl_all_gather_gemm, nccl_gemm_reduce_scatter

    M, H, F = a.tokens, a.hidden, a.ffn
    Ml, Fl = M // world, F // world
    ctx = TensorParallelContext(group, Ml, H, H, num_gpu_timeout_secs=20)
    g = torch.Generator(device='cuda').manual_seed(rank)
    x_shard = torch.randn((Ml, H), device=dev, generator=g).bfloat16()
    w1 = (torch.randn((Fl, H), device=dev, generator=g) * 0.02).bfloat16()
    x2 = torch.randn((M, Fl), device=dev, generator=g).bfloat16()
    w2 = (torch.randn((H, Fl), device=dev, generator=g) * 0.02).bfloat16()
    dummy = torch.ones(1, device=dev)

    def timeit(fn) -> float:
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(a.iters):
            torch.cuda.synchronize()
            torch.cuda._sleep(int(4e6))
            dist.all_reduce(dummy)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        t = torch.tensor([total / a.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def rel(x, y) -> float:
        return ((x.float() - y.float()).norm() / y.float().norm()).item()

    err1 = rel(ctx.all_gather_gemm(x_shard, w1), nccl_all_gather_gemm(x_shard, w1, group))
    err2 = rel(ctx.gemm_reduce_scatter(x2, w2), nccl_gemm_reduce_scatter(x2, w2, group))
    torch.cuda.synchronize()
    ctx.check_status()
    if rank == 0:
        print(f'world {world}, tokens {M}, hidden {H}, ffn {F}; pairs {os.environ.get("EP_TP_CTA_PAIR", "0")}: '
              f'rel err ag_gemm {err1:.2e} gemm_rs {err2:.2e}', flush=True)
    flops = 2 * M * Fl * H
    err_ce = rel(ctx.all_gather_gemm(x_shard, w1, push='ce'), nccl_all_gather_gemm(x_shard, w1, group))
    t = timeit(lambda: ctx.all_gather_gemm(x_shard, w1, push='ce'))
    if rank == 0:
        print(f'ag_gemm fused, shard pushed by the copy engines (all SMs on the GEMM): {t * 1e3:.1f} us  {flops / t / 1e9:.0f} TFLOP/s per GPU, '
              f'rel err {err_ce:.2e}', flush=True)
    for comm in [int(v) for v in a.comm_ctas.split(',')]:
        t = timeit(lambda: ctx.all_gather_gemm(x_shard, w1, num_comm_ctas=comm, push='sm'))
        if rank == 0:
            print(f'ag_gemm fused, {comm} push CTAs inside the kernel: {t * 1e3:.1f} us  {flops / t / 1e9:.0f} TFLOP/s per GPU', flush=True)
    tb = timeit(lambda: nccl_all_gather_gemm(x_shard, w1, group))
    gathered = torch.empty((M, H), device=dev, dtype=torch.bfloat16)
    tg = timeit(lambda: torch.matmul(gathered, w1.t()))
    t2 = timeit(lambda: ctx.gemm_reduce_scatter(x2, w2))
    tb2 = timeit(lambda: nccl_gemm_reduce_scatter(x2, w2, group))
    tg2 = timeit(lambda: torch.matmul(x2, w2.t()))
    if rank == 0:
        print(f'ag_gemm baseline NCCL all-gather + cuBLAS: {tb * 1e3:.1f} us (cuBLAS alone {tg * 1e3:.1f} us)')
        print(f'gemm_rs fused: {t2 * 1e3:.1f} us  {flops / t2 / 1e9:.0f} TFLOP/s per GPU | baseline cuBLAS + NCCL reduce-scatter: '
              f'{tb2 * 1e3:.1f} us (cuBLAS alone {tg2 * 1e3:.1f} us)', flush=True)
    ctx.check_status()
    dist.barrier()
    torch.cuda.synchronize()
    ctx.destroy()
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
