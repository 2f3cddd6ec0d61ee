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
