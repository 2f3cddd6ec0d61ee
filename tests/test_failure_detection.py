"""Failure detection without faulting a GPU. Host side: a rank that exits is noticed through the
store heartbeat (gloo / TCPStore processes on CPU). Device side (GPU tests): a wait that nothing
satisfies runs out after a short limit, the kernel returns, the host reads the status and raises;
in shrink mode the silent rank is masked and the survivors keep going."""
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _hb_worker(rank: int, world: int, port: int, result):
    from deepep_b200.utils.heartbeat import Heartbeat
    store = dist.TCPStore('127.0.0.1', port, world, is_master=(rank == 0), timeout=__import__('datetime').timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, interval=0.1, timeout=0.8)
    time.sleep(0.5)
    assert hb.dead_ranks() == []
    if rank == 1:
        hb.stop()           # rank 1 "dies" between steps: its beat stops advancing
        time.sleep(3.0)
        return
    deadline = time.time() + 6
    dead = []
    while time.time() < deadline and not dead:
        time.sleep(0.2)
        dead = hb.dead_ranks()
    result.put(dead)
    hb.stop()


def test_heartbeat_notices_a_rank_that_stops():
    ctx = mp.get_context('spawn')
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hb_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    dead = result.get(timeout=30)
    for p in procs:
        p.join(timeout=30)
    assert dead == [1]


class _DictStore:
    """The two methods of a ``torch.distributed`` store that the heartbeat uses."""

    def __init__(self):
        self.data = {}

    def set(self, key, value):
        self.data[key] = value

    def get(self, key):
        return self.data[key].encode()


def test_heartbeat_keeps_beating_while_a_native_call_blocks():
    """A healthy rank that sits in a long native wait (the drivers release the GIL for the host spin on the received
    counts and for stream synchronisation) must keep publishing its beat: otherwise the survivors of a real failure
    would take the waiting victim for dead as well. The wait is made on the host, no GPU is involved."""
    import deepep_b200
    from deepep_b200.utils.heartbeat import Heartbeat
    if deepep_b200._C is None:
        pytest.skip('native extension not built')
    store = _DictStore()
    hb = Heartbeat(store, 0, 2, interval=0.02, timeout=1.0)
    time.sleep(0.1)
    before = int(store.get('hb/0'))
    deepep_b200._C.debug_blocking_host_wait(0.6)        # ~30 beat intervals inside one native call
    after = int(store.get('hb/0'))
    hb.stop()
    assert after - before >= 10, f'the heartbeat advanced by only {after - before} during a blocking native call'


@pytest.mark.gpu
def test_device_wait_runs_out_and_reports():
    import deepep_b200
    from deepep_b200.parallel.local_cluster import LocalCluster
    cl = LocalCluster(2, num_max_tokens_per_rank=16, hidden=256, num_topk=2, num_gpu_timeout_secs=0.3)
    C = deepep_b200._C
    # only rank 0 enters the barrier: rank 1's arrival word is never written
    t0 = time.time()
    C.Runtime.barrier([cl.buffers[0].runtime], True, False)
    torch.cuda.synchronize()
    assert time.time() - t0 < 5
    with pytest.raises(deepep_b200.EPTimeoutError) as err:
        cl.buffers[0].check_status()
    assert 'barrier' in str(err.value) and 'peer 1' in str(err.value)
    cl.buffers[1].check_status()          # the other rank is healthy
    cl.destroy()
    # recovery = rebuild the buffers; the GPU context is intact
    cl2 = LocalCluster(2, num_max_tokens_per_rank=16, hidden=256, num_topk=2, num_gpu_timeout_secs=5)
    cl2.barrier(with_cpu_sync=True)
    cl2.destroy()


@pytest.mark.gpu
def test_low_latency_shrink_masks_a_silent_rank():
    import deepep_b200
    from deepep_b200.parallel.local_cluster import LocalCluster
    from conftest import make_routed_inputs
    C = deepep_b200._C
    R, T, H, E, K = 3, 8, 256, 6, 2
    cl = LocalCluster(R, num_bytes=deepep_b200.Buffer.get_low_latency_rdma_size_hint(T, H, R, E), num_gpu_timeout_secs=0.3)
    xs, idxs, ws = make_routed_inputs(R, T, H, E, K, seed=5, device='cuda', vary_tokens=False)
    survivors = cl.runtimes[:2]
    ios = []
    for r in range(2):
        io = C.LLDispatchIO()
        io.x, io.topk_idx = xs[r], idxs[r]
        ios.append(io)
    # rank 2 never launches: with shrink the survivors mask it after the short limit and finish
    C.ll_dispatch(survivors, ios, T, E, False, False, False, C.LL_SEND | C.LL_RECV, 4, True, False, True)
    torch.cuda.synchronize()
    for r in range(2):
        cl.buffers[r].check_status()       # shrink mode masks instead of reporting
        mask = torch.zeros(R, dtype=torch.int32, device='cuda')
        C.ll_mask_query(cl.runtimes[r], mask)
        assert mask.tolist() == [0, 0, 1]
    # rows that came from the survivors are intact
    EL = E // R
    for r in range(2):
        for le in range(EL):
            e = r * EL + le
            expect = sum(int((idxs[s] == e).sum()) for s in range(2))
            assert int(ios[r].packed_recv_count[le]) == expect
    # the next call does not wait for the masked rank at all
    t0 = time.time()
    C.ll_dispatch(survivors, ios, T, E, False, False, False, C.LL_SEND | C.LL_RECV, 4, True, False, True)
    torch.cuda.synchronize()
    assert time.time() - t0 < 0.25
    C.ll_mask_clean(cl.runtimes[0])
    cl.destroy()
