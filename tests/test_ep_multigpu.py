"""Real multi-process expert parallelism: one process per GPU, heaps exchanged as CUDA IPC
handles over the NCCL process group, results checked against the collective oracle.
Needs at least two GPUs (skipped otherwise). Modelled on tests/elastic/test_ep.py of the
reference, which spawns one process per GPU in the same way."""
import os
import socket

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, fused_fp8: bool):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    import deepep_b200
    from deepep_b200.utils import gate, refs
    from deepep_b200.utils.math import per_token_cast_to_fp8
    T, H, E, K = 256, 2048, 8 * world, 4
    buf = deepep_b200.ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=T, hidden=H, num_topk=K,
                                    num_gpu_timeout_secs=10, explicitly_destroy=True)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn((T - rank, H), generator=g).bfloat16().to(dev)
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(T - rank, E, generator=g), K, masked_ratio=0.05, generator=g)
    idx, w = idx.to(dev), w.to(dev)
    for it in range(3):
        if fused_fp8:
            (rx, rsf), ridx, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=8, fused_fp8=True)
            q = per_token_cast_to_fp8(x)
            (ex, esf), eidx, ew, esrc, _ = refs.dispatch(q, idx, w, T, E)
            assert torch.equal(rx.view(torch.uint8), ex.view(torch.uint8)) and torch.equal(rsf, esf)
            y = rx.float().bfloat16()
        else:
            rx, ridx, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=8)
            ex, eidx, ew, esrc, _ = refs.dispatch(x, idx, w, T, E)
            assert torch.equal(rx, ex)
            y = rx
        assert torch.equal(ridx, eidx) and torch.equal(rw, ew)
        assert torch.equal(handle.recv_src_metadata[:, 0], esrc)
        out, ow, _ = buf.combine(y, handle, topk_weights=rw)
        ref = refs.combine(y, handle.recv_src_metadata[:, 0], x.size(0), T)
        assert torch.equal(out, ref)
        buf.barrier(with_cpu_sync=True)
    buf.check_status()
    dist.barrier()
    buf.destroy()
    dist.destroy_process_group()


@pytest.mark.parametrize('fused_fp8', [False, True])
def test_two_or_more_gpus(fused_fp8):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs at least two GPUs')
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    torch.multiprocessing.spawn(_worker, args=(world, _free_port(), fused_fp8), nprocs=world, join=True)


def _subsystems_worker(rank: int, world: int, port: int):
    """Low-latency mode, AGRS, reduce-scatter, PP ring, Engram, fused TP GEMMs and the MoE module on real ranks."""
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    group = dist.group.WORLD
    import deepep_b200
    from deepep_b200.utils import gate
    g = torch.Generator().manual_seed(500 + rank)

    # ---- low-latency dispatch / combine through the legacy front end
    T, H, E, K = 32, 1024, 4 * world, 2
    EL = E // world
    ll = deepep_b200.Buffer(group, num_rdma_bytes=deepep_b200.Buffer.get_low_latency_rdma_size_hint(T, H, world, E),
                            low_latency_mode=True, num_gpu_timeout_secs=10, explicitly_destroy=True)
    x = torch.randn((T, H), generator=g).bfloat16().to(dev)
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K)
    idx, w = idx.to(dev), w.to(dev)
    for it in range(3):
        rx, cnt, handle, _, _ = ll.low_latency_dispatch(x, idx, T, E, use_fp8=False)
        # every received row must be the source row its src_info names
        all_x = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(all_x, x)
        for le in range(EL):
            n = int(cnt[le])
            info = handle[0][le, :n]
            lay = handle[1][le]
            begin = 0
            for s in range(world):
                c = int(lay[s]) & 0xffffffff
                tok = (info[begin:begin + c] & 0xffff).long()
                assert torch.equal(rx[le, begin:begin + c], all_x[s][tok])
                begin += c
        out, _, _ = ll.low_latency_combine(rx, idx, w, handle)
        valid_w = torch.where(idx >= 0, w, torch.zeros_like(w)).sum(dim=1, keepdim=True)
        assert torch.allclose(out.float(), x.float() * valid_w, rtol=2e-2, atol=2e-2)
        # LogFMT wire format: small rows are really encoded (result differs from bf16) and stay within its precision
        small = (rx.float() * 0.05).bfloat16()
        out_log, _, _ = ll.low_latency_combine(small, idx, w, handle, use_logfmt=True)
        want = x.float() * 0.05 * valid_w
        assert deepep_b200.utils.math.calc_diff(out_log.float(), want) < 2e-4
    ll.check_status()
    dist.barrier()
    ll.destroy()

    # ---- AGRS, reduce-scatter, PP, Engram on one elastic buffer
    buf = deepep_b200.ElasticBuffer(group, num_bytes=64 << 20, num_gpu_timeout_secs=10, explicitly_destroy=True)
    buf.agrs_set_config(4 << 20, 8)
    for it in range(2):
        with buf.agrs_new_session():
            t = torch.full((64, 32), float(rank + it), device=dev)
            gathered, wait = buf.all_gather(t)
            wait()
            assert torch.equal(gathered, torch.stack([torch.full((64, 32), float(r + it), device=dev) for r in range(world)]))
            z = torch.randn((world * 8, 64), generator=g).bfloat16().to(dev)
            rs = buf.reduce_scatter(z)
            ref = z.float().clone()
            dist.all_reduce(ref)
            assert torch.allclose(rs.float(), ref[rank * 8:(rank + 1) * 8], rtol=2e-2, atol=2e-2)
            torch.cuda.synchronize()
    buf.pp_set_config(1 << 16, 2)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for it in range(5):
        buf.pp_send(torch.full((1000,), float(rank * 10 + it), device=dev), nxt)
        got = torch.empty(1000, device=dev)
        buf.pp_recv(got, prv)
        assert torch.equal(got, torch.full((1000,), float(prv * 10 + it), device=dev))
    per_rank, hidden = 32, 128
    table = torch.arange(world * per_rank, device=dev).float().unsqueeze(1).expand(-1, hidden).bfloat16().contiguous()
    buf.engram_write(table[rank * per_rank:(rank + 1) * per_rank].contiguous())
    q = torch.randint(0, world * per_rank, (9, 2), device=dev, dtype=torch.int32)
    data, _ = buf.engram_fetch(q)()
    torch.cuda.synchronize()
    assert torch.equal(data, table[q.flatten().long()])
    buf.check_status()
    dist.barrier()
    buf.destroy()

    # ---- the same table in the ranks' pinned host segments (one POSIX shared-memory object per rank, read over PCIe)
    hbuf = deepep_b200.ElasticBuffer(group, num_bytes=16 << 20, num_cpu_bytes=1 << 20, num_gpu_timeout_secs=10, explicitly_destroy=True)
    assert len(hbuf.host_segments) == world
    hbuf.engram_write(table[rank * per_rank:(rank + 1) * per_rank].contiguous())
    data, _ = hbuf.engram_fetch(q)()
    torch.cuda.synchronize()
    assert torch.equal(data, table[q.flatten().long()])
    hbuf.check_status()
    dist.barrier()
    hbuf.destroy()

    # ---- fused tensor-parallel GEMMs against NCCL + matmul
    from deepep_b200.parallel.tp_fused import TensorParallelContext, nccl_all_gather_gemm, nccl_gemm_reduce_scatter
    ctx = TensorParallelContext(group, 256, 512, 512, num_gpu_timeout_secs=10)
    gc = torch.Generator(device='cuda').manual_seed(rank)
    for it in range(4):
        xs = torch.randn((256, 512), device=dev, generator=gc).bfloat16()
        w1 = (torch.randn((512, 512), device=dev, generator=gc) * 0.05).bfloat16()
        # the shard is pushed by CTAs of the kernel on even iterations and by the copy engines on odd ones: both use the
        # same gather halves and flag words, so they must also work interleaved
        a = ctx.all_gather_gemm(xs, w1, num_comm_ctas=2, num_sms=24, push='sm' if it % 2 == 0 else 'ce')
        b = nccl_all_gather_gemm(xs, w1, group)
        assert ((a.float() - b.float()).norm() / b.float().norm()).item() < 1e-2
        x2 = torch.randn((world * 256, 256), device=dev, generator=gc).bfloat16()
        w2 = (torch.randn((512, 256), device=dev, generator=gc) * 0.05).bfloat16()
        c = ctx.gemm_reduce_scatter(x2, w2, num_sms=24)
        d = nccl_gemm_reduce_scatter(x2, w2, group)
        assert ((c.float() - d.float()).norm() / d.float().norm()).item() < 2e-2
    torch.cuda.synchronize()
    ctx.check_status()
    dist.barrier()
    ctx.destroy()

    # ---- the MoE module: forward + backward runs and produces finite gradients on every rank
    from deepep_b200.models.moe import FusedMoE, MoEConfig
    Tm, Hm, Im, Em, Km = 64, 256, 128, 2 * world, 2
    mbuf = deepep_b200.ElasticBuffer(group, num_max_tokens_per_rank=Tm, hidden=Hm, num_topk=Km, num_gpu_timeout_secs=10, explicitly_destroy=True)
    layer = FusedMoE(mbuf, MoEConfig(hidden=Hm, intermediate=Im, num_experts=Em, num_topk=Km, num_sms=8))
    xm = torch.randn((Tm, Hm), generator=g).bfloat16().to(dev).requires_grad_(True)
    ym = layer(xm)
    (ym.float() ** 2).mean().backward()
    torch.cuda.synchronize()
    mbuf.check_status()
    for p in (xm, layer.router, layer.w13, layer.w2):
        assert p.grad is not None and torch.isfinite(p.grad.float()).all()
    dist.barrier()
    mbuf.destroy()
    dist.destroy_process_group()


def _digest(*tensors) -> str:
    import hashlib
    h = hashlib.sha256()
    for t in tensors:
        if t is None:
            continue
        t = t.contiguous()
        h.update(t.view(torch.uint8).cpu().numpy().tobytes())
    return h.hexdigest()


def _pressure_worker(rank: int, world: int, port: int, num_seeds: int):
    """Seed loop on real ranks, a new buffer per seed (tests/elastic/test_ep.py:387-404,547-557 of the reference): every
    seed draws a workload (token counts, masking, FP8 or bf16, plain or expanded), runs dispatch + combine twice and
    wants (a) the oracle's rows the first time and (b) the very same bits the second time."""
    import random
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    import deepep_b200
    from deepep_b200.utils import gate, refs
    from deepep_b200.utils.math import per_token_cast_to_fp8
    for seed in range(num_seeds):
        rng = random.Random(1000 + seed)                      # the same draw on every rank
        T = rng.choice([64, 200, 512])
        H = rng.choice([512, 2048, 7168])
        K = rng.choice([2, 4, 8])
        E = world * rng.choice([8, 16, 32])
        fp8 = rng.random() < 0.5
        expand = rng.random() < 0.4
        masked = rng.choice([0.0, 0.1, 0.5])
        sms = rng.choice([2, 6, 24])
        junk = torch.full((256 << 20,), 0xFF, dtype=torch.uint8, device=dev)      # poison what the allocator hands out next
        del junk
        buf = deepep_b200.ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=T, hidden=H, num_topk=K,
                                        num_gpu_timeout_secs=10, explicitly_destroy=True)
        g = torch.Generator().manual_seed(seed * 131 + rank)
        t = T - (rank * 7) % 23
        x = torch.randn((t, H), generator=g).bfloat16().to(dev)
        idx, w = gate.topk_from_scores(gate.get_balanced_scores(t, E, generator=g), K, masked_ratio=masked, generator=g)
        idx, w = idx.to(dev), w.to(dev)
        digests = []
        for run in range(2):
            kw = dict(topk_idx=idx, topk_weights=w, num_experts=E, num_sms=sms, do_expand=expand,
                      expert_alignment=16 if expand else 1, do_zero_padding=expand, fused_fp8=fp8)
            rx, ridx, rw, handle, _ = buf.dispatch(x, **kw)
            rxd, rsf = rx if fp8 else (rx, None)
            y = torch.randn(rxd.shape, generator=torch.Generator().manual_seed(seed + 7 * rank)).bfloat16().to(dev)
            out, ow, _ = buf.combine(y, handle, topk_weights=rw)
            torch.cuda.synchronize()
            buf.check_status()
            digests.append(_digest(rxd, rsf, ridx, rw, handle.recv_src_metadata, out, ow))
            if run == 0 and not expand:
                src = per_token_cast_to_fp8(x) if fp8 else x
                ex, eidx, ew, esrc, _ = refs.dispatch(src, idx, w, T, E)
                if fp8:
                    assert torch.equal(rxd.view(torch.uint8), ex[0].view(torch.uint8)) and torch.equal(rsf, ex[1])
                else:
                    assert torch.equal(rxd, ex)
                assert torch.equal(ridx, eidx) and torch.equal(rw, ew) and torch.equal(handle.recv_src_metadata[:, 0], esrc)
                assert torch.equal(out, refs.combine(y, esrc, t, T))
        assert digests[0] == digests[1], f'seed {seed}: two runs of the same workload differ'
        dist.barrier()
        buf.destroy()
    dist.destroy_process_group()


def test_pressure_seed_loop_on_real_ranks():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs at least two GPUs')
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    torch.multiprocessing.spawn(_pressure_worker, args=(world, _free_port(), 8), nprocs=world, join=True)


def _ll_graph_worker(rank: int, world: int, port: int):
    """The low-latency pair captured in ONE CUDA graph and replayed with new tokens every time; every replay is checked."""
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    import deepep_b200
    from deepep_b200.utils import gate
    T, H, E, K = 64, 2048, 8 * world, 4
    ll = deepep_b200.Buffer(dist.group.WORLD, num_rdma_bytes=deepep_b200.Buffer.get_low_latency_rdma_size_hint(T, H, world, E),
                            low_latency_mode=True, num_gpu_timeout_secs=10, explicitly_destroy=True)
    g = torch.Generator().manual_seed(77 + rank)
    x = torch.randn((T, H), generator=g).bfloat16().to(dev)
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K, masked_ratio=0.1, generator=g)
    idx, w = idx.to(dev), w.to(dev)
    out = torch.empty_like(x)

    def step():
        rx, cnt, handle, _, _ = ll.low_latency_dispatch(x, idx, T, E, use_fp8=False)
        ll.low_latency_combine(rx, idx, w, handle, out=out)      # identity experts

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    valid_w = torch.where(idx >= 0, w, torch.zeros_like(w)).sum(dim=1, keepdim=True)
    for it in range(12):
        x.copy_(torch.randn((T, H), generator=g).bfloat16())     # new tokens, same graph
        graph.replay()
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), x.float() * valid_w, rtol=2e-2, atol=2e-2), f'replay {it}'
    ll.check_status()
    dist.barrier()
    ll.destroy()
    dist.destroy_process_group()


def test_low_latency_graph_replay_on_real_ranks():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs at least two GPUs')
    world = 4 if n >= 4 else 2
    torch.multiprocessing.spawn(_ll_graph_worker, args=(world, _free_port()), nprocs=world, join=True)


def _backend_worker(rank: int, world: int, port: int):
    """The virtual-memory heap (cuMemCreate + descriptors passed over a unix socket) with a pinned CPU segment in the same
    address range, and flag rounds as stream memory operations: dispatch / combine, an Engram table in the CPU
    segments, and an all-gather session must give the same results as with the default heap."""
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    os.environ['EP_HEAP_BACKEND'] = 'vmm'
    os.environ['EP_STREAM_MEMOPS'] = '1'
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    import deepep_b200
    from deepep_b200.utils import gate, refs
    T, H, E, K = 128, 1024, 8 * world, 4
    buf = deepep_b200.ElasticBuffer(dist.group.WORLD, num_max_tokens_per_rank=T, hidden=H, num_topk=K, num_cpu_bytes=1 << 20,
                                    num_gpu_timeout_secs=10, explicitly_destroy=True)
    assert buf.heap_is_vmm and len(buf.host_segments) == world
    g = torch.Generator().manual_seed(900 + rank)
    x = torch.randn((T, H), generator=g).bfloat16().to(dev)
    idx, w = gate.topk_from_scores(gate.get_balanced_scores(T, E, generator=g), K)
    idx, w = idx.to(dev), w.to(dev)
    for it in range(2):
        rx, ridx, rw, handle, _ = buf.dispatch(x, topk_idx=idx, topk_weights=w, num_experts=E, num_sms=8)
        ex, eidx, ew, esrc, _ = refs.dispatch(x, idx, w, T, E)
        assert torch.equal(rx, ex) and torch.equal(ridx, eidx)
        out, _, _ = buf.combine(rx, handle)
        assert torch.equal(out, refs.combine(rx, esrc, T, T))
    # Engram rows served from the ranks' CPU segments (behind the GPU segment in the same window)
    per_rank, hidden = 32, 128
    table = torch.arange(world * per_rank, device=dev).float().unsqueeze(1).expand(-1, hidden).bfloat16().contiguous()
    buf.engram_write(table[rank * per_rank:(rank + 1) * per_rank].contiguous())
    q = torch.randint(0, world * per_rank, (9, 2), device=dev, dtype=torch.int32)
    data, _ = buf.engram_fetch(q)()
    torch.cuda.synchronize()
    assert torch.equal(data, table[q.flatten().long()])
    buf.check_status()
    dist.barrier()
    buf.destroy()
    # an all-gather session whose arrival rounds are stream memory operations (no kernel, no SM)
    assert deepep_b200._C.stream_memops_enabled()
    abuf = deepep_b200.ElasticBuffer(dist.group.WORLD, num_bytes=32 << 20, num_gpu_timeout_secs=10, explicitly_destroy=True)
    abuf.agrs_set_config(1 << 20, 4)
    for it in range(3):
        with abuf.agrs_new_session():
            t = torch.full((256, 64), float(rank * 3 + it), device=dev)
            gathered, wait = abuf.all_gather(t)
            wait()
            assert torch.equal(gathered, torch.stack([torch.full((256, 64), float(r * 3 + it), device=dev) for r in range(world)]))
            torch.cuda.synchronize()
    dist.barrier()
    abuf.destroy()
    dist.destroy_process_group()


def test_vmm_heap_and_stream_memops_on_real_ranks():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs at least two GPUs')
    torch.multiprocessing.spawn(_backend_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_subsystems_on_real_ranks():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip('needs at least two GPUs')
    world = 4 if n >= 4 else 2
    torch.multiprocessing.spawn(_subsystems_worker, args=(world, _free_port()), nprocs=world, join=True)
