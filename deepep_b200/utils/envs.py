"""Environment and topology probes, process-group bootstrap, seeding.

Parity: deep_ep/utils/envs.py:24-268 of the reference. There is one tier here (the NVLink /
NVSwitch domain of one box), so the "physical" and "logical" domains are both
``(1, world_size)`` and the RDMA probes report "no RDMA tier".
"""
from __future__ import annotations

import os
import re
import subprocess
from typing import Optional, Tuple

import torch
import torch.distributed as dist

_GLOBAL_SEED = 0
_LOCAL_SEED = 0

# Nominal NVLink 5 figures of a B200 (18 links x 50 GB/s per direction).
NVLINK5_LINKS = 18
NVLINK5_GBS_PER_LINK = 50.0


def init_seed(global_seed: int) -> None:
    """Seeds torch with a rank-dependent local seed and remembers both seeds."""
    global _GLOBAL_SEED, _LOCAL_SEED
    rank = dist.get_rank() if dist.is_initialized() else 0
    _GLOBAL_SEED = global_seed
    _LOCAL_SEED = global_seed * 1024 + rank
    torch.manual_seed(_LOCAL_SEED)


def get_local_seed() -> int:
    return _LOCAL_SEED


def get_global_seed() -> int:
    return _GLOBAL_SEED


def dist_print(s: str = '', once_in_node: bool = False) -> None:
    """Prints from every rank in rank order, or only from rank 0 with ``once_in_node``."""
    if not dist.is_initialized():
        print(s, flush=True)
        return
    rank, world = dist.get_rank(), dist.get_world_size()
    if once_in_node:
        if rank == 0:
            print(s, flush=True)
        dist.barrier()
        return
    for r in range(world):
        if r == rank:
            print(s, flush=True)
        dist.barrier()


def init_dist(local_rank: int, num_local_ranks: int, seed: int = 0, backend: Optional[str] = None
              ) -> Tuple[int, int, dist.ProcessGroup]:
    """Joins the default process group of a single-node job and returns ``(rank, world, group)``.

    Reads ``MASTER_ADDR`` (default 127.0.0.1) and ``MASTER_PORT`` (default 8361). With CUDA available
    the backend is NCCL and the process binds to ``cuda:local_rank``; otherwise gloo on CPU.
    """
    addr = os.environ.get('MASTER_ADDR', '127.0.0.1')
    port = int(os.environ.get('MASTER_PORT', '8361'))
    use_cuda = torch.cuda.is_available()
    backend = backend or ('nccl' if use_cuda else 'gloo')
    kwargs = {}
    if use_cuda:
        torch.cuda.set_device(local_rank)
        if backend == 'nccl':
            kwargs['device_id'] = torch.device('cuda', local_rank)
    dist.init_process_group(backend=backend, init_method=f'tcp://{addr}:{port}', world_size=num_local_ranks,
                            rank=local_rank, **kwargs)
    if use_cuda:
        torch.set_default_device('cuda')
    init_seed(seed)
    group = dist.new_group(list(range(num_local_ranks)))
    return dist.get_rank(), num_local_ranks, group


def get_physical_domain_size(group: dist.ProcessGroup) -> Tuple[int, int]:
    """(RDMA ranks, NVLink ranks) — one box: every rank is an NVLink peer."""
    return 1, group.size()


def get_logical_domain_size(group: dist.ProcessGroup, allow_hybrid_mode: bool = True) -> Tuple[int, int]:
    """(scale-out ranks, scale-up ranks) — one tier, whatever ``allow_hybrid_mode`` says."""
    return 1, group.size()


def check_nvlink_connections(group: dist.ProcessGroup) -> None:
    """Asserts that every pair of the group's GPUs can reach each other's memory (P2P)."""
    if not torch.cuda.is_available() or group.size() == 1:
        return
    me = torch.cuda.current_device()
    devices = [None] * group.size()
    dist.all_gather_object(devices, me, group=group)
    for other in devices:
        if other != me and other < torch.cuda.device_count():
            assert torch.cuda.can_device_access_peer(me, other), f'GPU {me} cannot access GPU {other} over P2P'


def check_torch_deterministic() -> None:
    """Deterministic fill of uninitialised memory would clobber buffers that peers write into."""
    if torch.are_deterministic_algorithms_enabled():
        assert not torch.utils.deterministic.fill_uninitialized_memory, \
            'disable torch.utils.deterministic.fill_uninitialized_memory when using this library'


def parse_nvlink_status(text: str) -> Tuple[int, float]:
    """(number of links, GB/s per link) from ``nvidia-smi nvlink -s`` output of one GPU."""
    speeds = [float(v) for v in re.findall(r'Link\s+\d+:\s+([0-9.]+)\s+GB/s', text)]
    if not speeds:
        return 0, 0.0
    return len(speeds), sum(speeds) / len(speeds)


def get_nvlink_gbs(factor: float = 0.9) -> float:
    """Usable NVLink bandwidth per direction of the current GPU in GB/s (nominal x ``factor``).

    Parsed from ``nvidia-smi nvlink -s``; falls back to the NVLink 5 figures (18 x 50 GB/s).
    """
    links, per_link = 0, 0.0
    try:
        idx = torch.cuda.current_device() if torch.cuda.is_available() else 0
        out = subprocess.run(['nvidia-smi', 'nvlink', '-s', '-i', str(idx)], capture_output=True, text=True, timeout=10)
        links, per_link = parse_nvlink_status(out.stdout)
    except (OSError, subprocess.SubprocessError):
        pass
    if links == 0:
        links, per_link = NVLINK5_LINKS, NVLINK5_GBS_PER_LINK
    return links * per_link * factor


def check_fast_rdma_atomic_support(nic_name: str = '') -> bool:
    """No RDMA tier on a single box."""
    return False


def get_rdma_gbs(nic_name: str = '') -> float:
    """No RDMA tier on a single box."""
    return 0.0
