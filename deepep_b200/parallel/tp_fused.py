"""Tensor-parallel linear layers whose GEMM is fused with its collective.

``TensorParallelContext`` owns a symmetric heap and exposes

* ``all_gather_gemm(x_shard, w_shard)``: ``gather_ranks(x_shard)[R * Ml, K] @ w_shard[N, K].T`` — the
  column-parallel linear that follows a sequence/token-sharded activation;
* ``gemm_reduce_scatter(x, w_shard)``: ``reduce_scatter_rows(x[R * Ml, Kl] @ w_shard[N, Kl].T)`` — the
  row-parallel linear whose output is sharded by token again.

Both run as ONE sm_100a kernel per rank (tcgen05 main loop + peer stores / flags over NVLink), see
``csrc/kernels/tp_fused.cu``. The reference library has no counterpart (it stops at a copy-engine
all-gather); the baselines are ``dist.all_gather_into_tensor`` + matmul and matmul +
``dist.reduce_scatter_tensor``, available here as :func:`nccl_all_gather_gemm` /
:func:`nccl_gemm_reduce_scatter`.
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence

import torch
import torch.distributed as dist

from .._native import _C, require_native
from ..buffers.elastic import ElasticBuffer


def _align(x: int, a: int = 256) -> int:
    return -(-x // a) * a


class TensorParallelContext:
    """Buffer + offsets for the fused operators of one tensor-parallel group.

    Arguments:
        group: process group (or a virtual rank of a ``LocalCluster``-style emulation).
        rows_per_rank: token rows every rank owns (multiple of 128).
        gather_k: reduction dimension of the all-gather -> GEMM (width of the gathered activation).
        scatter_n: output width of the GEMM -> reduce-scatter.
    """

    def __init__(self, group: Any, rows_per_rank: int, gather_k: int, scatter_n: int, num_gpu_timeout_secs: float = 30):
        require_native()
        assert rows_per_rank % 128 == 0
        R = group.size()
        self.group, self.num_ranks, self.rows_per_rank = group, R, rows_per_rank
        ctl = int(_C.CONTROL_BYTES)
        gather_half = _align(R * rows_per_rank * gather_k * 2)
        part_half = _align(R * rows_per_rank * scatter_n * 2)
        flag_half = _align(R * (rows_per_rank // 128) * max(scatter_n // 256, 1) * 8)
        self.gather_offsets = [ctl, ctl + gather_half]
        base = ctl + 2 * gather_half
        self.partial_offsets = [base, base + part_half]
        base += 2 * part_half
        self.flag_offsets = [base, base + flag_half]
        total = base + 2 * flag_half
        align = ElasticBuffer.get_elastic_buffer_alignment()
        self.buffer = ElasticBuffer(group, num_bytes=-(-total // align) * align, num_gpu_timeout_secs=num_gpu_timeout_secs,
                                    explicitly_destroy=True)
        self.runtime = self.buffer.runtime

    def all_gather_gemm(self, x_shard: torch.Tensor, w_shard: torch.Tensor, num_comm_ctas: int = 0, num_sms: int = 0,
                        push: str = 'auto') -> torch.Tensor:
        """``push``: how the shard reaches the peers while the GEMM runs. ``'sm'``: push CTAs inside the kernel (bulk
        stores); ``'ce'``: copy engines on side streams with a stream-ordered flag write per row chunk, all SMs stay
        with the GEMM; ``'auto'`` (also ``EP_TP_PUSH=sm|ce``): copy engines where the driver offers stream writes."""
        mode = {'auto': 0, 'sm': 1, 'ce': 2}[push]
        return _C.tp_ag_gemm([self.runtime], [x_shard], [w_shard], self.gather_offsets, num_comm_ctas, num_sms, mode)[0]

    def gemm_reduce_scatter(self, x: torch.Tensor, w_shard: torch.Tensor, num_sms: int = 0) -> torch.Tensor:
        return _C.tp_gemm_rs([self.runtime], [x], [w_shard], self.partial_offsets, self.flag_offsets, num_sms)[0]

    def check_status(self) -> None:
        self.buffer.check_status()
        code = _C.tp_check_status()
        if code != 0:
            raise RuntimeError(f'a fused tensor-parallel kernel gave up waiting (status {code})')

    def destroy(self) -> None:
        self.buffer.destroy()


def fused_multi(contexts: Sequence[TensorParallelContext], op: str, xs: Sequence[torch.Tensor], ws: Sequence[torch.Tensor],
                **kw) -> List[torch.Tensor]:
    """Single-GPU emulation: all virtual ranks of ``contexts`` in one cooperative launch."""
    rts = [c.runtime for c in contexts]
    c0 = contexts[0]
    if op == 'ag_gemm':
        return _C.tp_ag_gemm(rts, list(xs), list(ws), c0.gather_offsets, kw.get('num_comm_ctas', 0), kw.get('num_sms', 0))
    return _C.tp_gemm_rs(rts, list(xs), list(ws), c0.partial_offsets, c0.flag_offsets, kw.get('num_sms', 0))


def nccl_all_gather_gemm(x_shard: torch.Tensor, w_shard: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Baseline: NCCL all-gather, then a library GEMM."""
    world = dist.get_world_size(group)
    full = torch.empty((world * x_shard.size(0), x_shard.size(1)), dtype=x_shard.dtype, device=x_shard.device)
    dist.all_gather_into_tensor(full, x_shard.contiguous(), group=group)
    return full @ w_shard.t()


def nccl_gemm_reduce_scatter(x: torch.Tensor, w_shard: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Baseline: a library GEMM, then NCCL reduce-scatter."""
    world = dist.get_world_size(group)
    partial = x @ w_shard.t()
    out = torch.empty((partial.size(0) // world, partial.size(1)), dtype=partial.dtype, device=partial.device)
    dist.reduce_scatter_tensor(out, partial, group=group)
    return out
