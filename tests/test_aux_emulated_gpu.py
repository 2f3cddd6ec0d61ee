"""AGRS sessions (all-gather, in-place, batched, reduce-scatter), PP slot rings and Engram with
emulated ranks on one GPU. Follows tests/elastic/test_agrs.py, test_pp.py and test_engram.py of the
reference: random op sequences checked against direct tensor algebra."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(R, num_bytes, num_cpu_bytes=0):
    import deepep_b200
    from deepep_b200.parallel.local_cluster import VirtualRanks
    vr = VirtualRanks(R)
    bufs = [deepep_b200.ElasticBuffer(vr.groups[r], num_bytes=num_bytes, num_cpu_bytes=num_cpu_bytes, num_gpu_timeout_secs=5)
            for r in range(R)]
    vr.connect()
    return bufs


def test_agrs_sessions():
    from deepep_b200.parallel.agrs import AgrsManager
    R = 4
    bufs = _buffers(R, 64 << 20)
    mgrs = [b._agrs_manager() for b in bufs]
    g = torch.Generator(device='cuda').manual_seed(0)
    for session in range(3):
        for m in mgrs:
            m.create_session()
        # plain all-gather
        xs = [torch.randn((33, 100), device='cuda', generator=g).bfloat16() for _ in range(R)]
        out = AgrsManager.multi_all_gather(mgrs, xs)
        for r in range(R):
            gathered, handle = out[r]
            handle()
            assert torch.equal(gathered, torch.stack(xs))
        # in-place + batched
        ys = []
        for r, m in enumerate(mgrs):
            a, b = m.get_inplace_tensor(((8, 64), (16,)), torch.float32)
            a.copy_(torch.full((8, 64), float(r + session)))
            b.copy_(torch.arange(16, device='cuda') * (r + 1.0))
            ys.append((a, b))
        out = AgrsManager.multi_all_gather(mgrs, ys)
        for r in range(R):
            ga, gb, handle = out[r]
            handle()
            assert torch.equal(ga, torch.stack([y[0] for y in ys])) and torch.equal(gb, torch.stack([y[1] for y in ys]))
        # reduce-scatter inside the session
        zs = [torch.randn((R * 16, 64), device='cuda', generator=g).bfloat16() for _ in range(R)]
        rs = AgrsManager.multi_reduce_scatter(mgrs, zs)
        total = torch.stack([z.float() for z in zs]).sum(dim=0)
        for r in range(R):
            assert torch.allclose(rs[r].float(), total[r * 16:(r + 1) * 16], rtol=2e-2, atol=2e-2)
        torch.cuda.synchronize()
        AgrsManager.multi_destroy(mgrs)
    torch.cuda.synchronize()
    for b in bufs:
        b.check_status()
        b.destroy()


def test_pp_ring_random_schedule():
    from deepep_b200.parallel.pp import PipelineRing
    R, slots = 4, 3
    bufs = _buffers(R, 32 << 20)
    rings = [b._pp_ring() for b in bufs]
    for ring in rings:
        ring.set_config(1 << 16, slots)
    g = torch.Generator().manual_seed(1)
    sent = []
    # forward wave: every rank sends `slots` tensors to its next rank before anything is received
    for i in range(slots):
        ts = [torch.full((1000,), float(10 * r + i), device='cuda') for r in range(R)]
        PipelineRing.multi_send(rings, ts, [(r + 1) % R for r in range(R)])
        sent.append(ts)
    for i in range(slots):
        outs = [torch.empty(1000, device='cuda') for _ in range(R)]
        PipelineRing.multi_recv(rings, outs, [(r - 1) % R for r in range(R)])
        torch.cuda.synchronize()
        for r in range(R):
            assert torch.equal(outs[r], sent[i][(r - 1) % R])
    # backward wave interleaved with forward sends, more rounds than slots
    for i in range(2 * slots):
        ts = [torch.full((512,), float(100 * r + i), device='cuda') for r in range(R)]
        PipelineRing.multi_send(rings, ts, [(r - 1) % R for r in range(R)])
        outs = [torch.empty(512, device='cuda') for _ in range(R)]
        PipelineRing.multi_recv(rings, outs, [(r + 1) % R for r in range(R)])
        torch.cuda.synchronize()
        for r in range(R):
            assert torch.equal(outs[r], ts[(r + 1) % R])
    for b in bufs:
        b.check_status()
        b.destroy()


@pytest.mark.parametrize('on_host', [False, True])
@pytest.mark.parametrize('fp8', [False, True])
def test_engram_fetch(fp8, on_host):
    """`on_host`: the shards live in the ranks' pinned host segments (num_cpu_bytes) and are fetched over PCIe."""
    from deepep_b200.parallel.engram import EngramStore
    R, per_rank, hidden = 4, 64, 256
    bufs = _buffers(R, 16 << 20, num_cpu_bytes=(1 << 20) if on_host else 0)
    stores = [b._engram_store() for b in bufs]
    assert all(s.on_host == on_host for s in stores)
    g = torch.Generator(device='cuda').manual_seed(2)
    table = torch.randn((R * per_rank, hidden), device='cuda', generator=g).bfloat16()
    sf = torch.rand((R * per_rank, 2), device='cuda', generator=g) if fp8 else None
    full = table.to(torch.float8_e4m3fn) if fp8 else table
    for r, s in enumerate(stores):
        s.write(full[r * per_rank:(r + 1) * per_rank].contiguous(), sf, barrier=False)
    torch.cuda.synchronize()
    idx = [torch.randint(0, R * per_rank, (17, 3), device='cuda', generator=g, dtype=torch.int32) for _ in range(R)]
    hooks = EngramStore.multi_fetch(stores, idx, col_major_sf=fp8)
    for r in range(R):
        data, got_sf = hooks[r]()
        torch.cuda.synchronize()
        flat = idx[r].flatten().long()
        assert torch.equal(data.view(torch.uint8) if fp8 else data, (full[flat].view(torch.uint8) if fp8 else full[flat]))
        if fp8:
            assert torch.equal(got_sf, sf[flat].view(17, 6))
            assert got_sf.stride(0) == 1
    if on_host:     # the table really is in host memory
        seg = bufs[1].host_segments[1].as_tensor()
        want = full[per_rank:2 * per_rank].contiguous().view(torch.uint8).flatten().cpu()
        assert torch.equal(seg[:want.numel()], want)
    for b in bufs:
        b.check_status()
        b.destroy()
