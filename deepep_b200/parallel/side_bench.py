"""Multi-GPU micro-benchmark of the side primitives: the copy-engine all-gather (AGRS), reduce-scatter, the
pipeline send / recv ring, the Engram table fetch (GPU and pinned-host segments) and the GPU barrier.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 \\
        -m deepep_b200.parallel.side_bench

Every figure is a CUDA-event time on the launching stream (several calls between two events where one call is
short; the stream is held back by a short sleep kernel first, so the calls are queued when the clock starts and
the figure is device time, not the host's launch time), maximum over ranks. NCCL collectives of the same shape are timed next to each primitive as the baseline.
Rank 0 prints one JSON line per primitive. Modelled on the bandwidth sweeps at the end of the reference's
tests/elastic/test_agrs.py:156-187, test_pp.py, test_engram.py and test_barrier.py.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--sizes-mb', default='1,4,16,64', help='per-rank payload of the all-gather / reduce-scatter sweep')
    ap.add_argument('--iters', type=int, default=10)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1)), int(os.environ.get('LOCAL_RANK', 0))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    dist.init_process_group('nccl', device_id=dev)
    group = dist.group.WORLD
    import deepep_b200
    _C = deepep_b200._C

    def max_over_ranks(v: float) -> float:
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timeit(fn, calls: int = 1) -> float:
        """Mean milliseconds of one call."""
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        total = 0.0
        for _ in range(a.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(int(1e6))     # the host queues the calls while the device idles: device time, not launch time
            e0.record()
            for _ in range(calls):
                fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1) / calls
        return max_over_ranks(total / a.iters)

    def emit(obj) -> None:
        if rank == 0:
            print(json.dumps(obj), flush=True)

    sizes = [int(float(v) * (1 << 20)) for v in a.sizes_mb.split(',')]
    largest = max(sizes)
    buf = deepep_b200.ElasticBuffer(group, num_bytes=deepep_b200.ElasticBuffer.get_agrs_buffer_size_hint(group, 2 * largest),
                                    num_gpu_timeout_secs=20, explicitly_destroy=True)
    memops = bool(_C.stream_memops_enabled())

    # ---------------------------------------------------------------- barrier
    ms = timeit(lambda: buf.barrier(), calls=50)
    ms_nccl = timeit(lambda: dist.barrier(), calls=10)
    emit({'op': 'barrier', 'world': world, 'us': round(ms * 1e3, 2), 'nccl_barrier_us': round(ms_nccl * 1e3, 2)})

    # ---------------------------------------------------------------- all-gather / reduce-scatter sweep
    for nbytes in sizes:
        n = nbytes // 2
        x = torch.randn(n, device=dev).bfloat16()
        out = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
        buf.agrs_set_config(2 * nbytes, 4)

        def ag():
            with buf.agrs_new_session():
                gathered, wait = buf.all_gather(x)
                wait()

        ms = timeit(ag)
        ms_nccl = timeit(lambda: dist.all_gather_into_tensor(out, x))
        with buf.agrs_new_session():
            gathered, wait = buf.all_gather(x)
            wait()
            dist.all_gather_into_tensor(out, x)
            ok = bool(torch.equal(gathered.flatten(), out))
            torch.cuda.synchronize()
        recv = (world - 1) * nbytes
        emit({'op': 'all_gather', 'world': world, 'mb_per_rank': nbytes / (1 << 20), 'us': round(ms * 1e3, 1), 'gbs_in': round(recv / ms / 1e6, 1),
              'nccl_us': round(ms_nccl * 1e3, 1), 'nccl_gbs_in': round(recv / ms_nccl / 1e6, 1), 'matches_nccl': ok,
              'signalling': 'stream memory operations (0 SMs)' if memops else 'one-block flag kernel'})

        z = torch.randn(world * (n // world), device=dev).bfloat16()
        rs_out = torch.empty(n // world, device=dev, dtype=torch.bfloat16)

        def rs():
            with buf.agrs_new_session():
                return buf.reduce_scatter(z)

        ms = timeit(rs)
        ms_nccl = timeit(lambda: dist.reduce_scatter_tensor(rs_out, z))
        got = rs()
        dist.reduce_scatter_tensor(rs_out, z)
        err = ((got.float() - rs_out.float()).norm() / rs_out.float().norm().clamp(min=1e-6)).item()
        sent = (world - 1) * (z.numel() // world) * 2
        emit({'op': 'reduce_scatter', 'world': world, 'mb_per_rank': z.numel() * 2 / (1 << 20), 'us': round(ms * 1e3, 1),
              'gbs_out': round(sent / ms / 1e6, 1), 'nccl_us': round(ms_nccl * 1e3, 1), 'nccl_gbs_out': round(sent / ms_nccl / 1e6, 1),
              'rel_err_vs_nccl': round(max_over_ranks(err), 5)})
    buf.check_status()
    dist.barrier()
    buf.destroy()

    # ---------------------------------------------------------------- pipeline ring
    pp_bytes = 32 << 20
    pbuf = deepep_b200.ElasticBuffer(group, num_bytes=deepep_b200.ElasticBuffer.get_pp_buffer_size_hint(pp_bytes, 2),
                                     num_gpu_timeout_secs=20, explicitly_destroy=True)
    pbuf.pp_set_config(pp_bytes, 2)
    t_send = torch.randn(pp_bytes // 2, device=dev).bfloat16()
    t_recv = torch.empty_like(t_send)
    nxt, prv = (rank + 1) % world, (rank - 1) % world

    def pp():
        pbuf.pp_send(t_send, nxt)
        pbuf.pp_recv(t_recv, prv)

    ms = timeit(pp)
    reqs = lambda: [dist.P2POp(dist.isend, t_send, nxt), dist.P2POp(dist.irecv, t_recv, prv)]

    def nccl_pp():
        for r in dist.batch_isend_irecv(reqs()):
            r.wait()

    ms_nccl = timeit(nccl_pp)
    emit({'op': 'pp_send_recv', 'world': world, 'mb': pp_bytes / (1 << 20), 'us': round(ms * 1e3, 1), 'gbs_per_direction': round(pp_bytes / ms / 1e6, 1),
          'nccl_send_recv_us': round(ms_nccl * 1e3, 1), 'nccl_gbs_per_direction': round(pp_bytes / ms_nccl / 1e6, 1)})
    pbuf.check_status()
    dist.barrier()
    pbuf.destroy()

    # ---------------------------------------------------------------- Engram fetch: GPU segment, then pinned-host segment
    entries_per_rank, hidden, tokens, per_token = 16384, 2048, 4096, 4
    table = torch.randn((entries_per_rank, hidden), device=dev).bfloat16()
    idx = torch.randint(0, world * entries_per_rank, (tokens, per_token), device=dev, dtype=torch.int32)
    for on_host in (False, True):
        store_bytes = deepep_b200.ElasticBuffer.get_engram_storage_size_hint(world * entries_per_rank, hidden, torch.bfloat16, world)
        kw = dict(num_cpu_bytes=entries_per_rank * hidden * 2) if on_host else {}
        try:
            ebuf = deepep_b200.ElasticBuffer(group, num_bytes=store_bytes if not on_host else 16 << 20, num_gpu_timeout_secs=20,
                                             explicitly_destroy=True, **kw)
        except Exception as exc:   # noqa: BLE001 - e.g. /dev/shm too small for the host segment
            emit({'op': 'engram_fetch', 'segment': 'host' if on_host else 'gpu', 'error': f'{type(exc).__name__}: {exc}'[:200]})
            continue
        ebuf.engram_write(table)

        def fetch():
            hook = ebuf.engram_fetch(idx)
            return hook()

        ms = timeit(fetch)
        data, _ = fetch()
        everyone = [torch.empty_like(table) for _ in range(world)]
        dist.all_gather(everyone, table)
        ok = bool(torch.equal(data, torch.cat(everyone)[idx.flatten().long()]))
        rows = tokens * per_token
        emit({'op': 'engram_fetch', 'segment': 'host' if on_host else 'gpu', 'world': world, 'rows': rows, 'row_bytes': hidden * 2,
              'us': round(ms * 1e3, 1), 'mrows_per_s': round(rows / ms / 1e3, 2), 'gbs': round(rows * hidden * 2 / ms / 1e6, 1), 'matches_all_gather': ok,
              'heap_backend': 'vmm (one address range)' if ebuf.heap_is_vmm else 'ipc (+ separate host mapping)'})
        ebuf.check_status()
        dist.barrier()
        ebuf.destroy()
        del everyone
    dist.destroy_process_group()


if __name__ == '__main__':
    main()
