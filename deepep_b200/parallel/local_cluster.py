"""Single-GPU emulation of a multi-rank expert-parallel job.

Kernels of different ranks wait on one another, so they cannot run as separate launches on one
GPU. ``LocalCluster`` instead creates ``num_ranks`` buffers in ONE process on ONE device, points
their peer tables at each other, and issues every collective operation as a single cooperative
launch in which blocks ``[v * num_sms, (v + 1) * num_sms)`` act as rank ``v``. The device code is
exactly the production code; only the peer pointers are local. This is what lets the multi-rank
logic (count exchange, prefix sums, slot placement, reduction order) be tested on a one-GPU box.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .._native import require_native
from ..buffers.elastic import ElasticBuffer
from ..utils.event import EventOverlap


class LocalGroup:
    """Stand-in for a process group: one virtual rank of a :class:`LocalCluster`."""

    is_local_emulation = True

    def __init__(self, cluster: 'LocalCluster', rank: int):
        self._cluster = cluster
        self._rank = rank

    def rank(self) -> int:
        return self._rank

    def size(self) -> int:
        return self._cluster.num_ranks

    def register(self, buffer) -> None:
        self._cluster._register(self._rank, buffer)


def _share_host_segments(buffers) -> None:
    """One process holds all ranks: every buffer sees the others' host segments through the same mappings."""
    if all(getattr(b, 'host_segments', None) for b in buffers) and all(hasattr(b, 'runtime') for b in buffers):
        own = [b.host_segments[0] for b in buffers]
        for b in buffers:
            b.host_segments = list(own)


class LocalCluster:
    """``num_ranks`` virtual ranks on the current device.

    ``buffers[r]`` is a regular :class:`ElasticBuffer`; the collective methods of the cluster take
    one argument list per rank and return one result per rank.
    """

    def __init__(self, num_ranks: int, **buffer_kwargs):
        self._C = require_native()
        assert 1 <= num_ranks <= self._C.MAX_VRANKS
        self.num_ranks = num_ranks
        self._pending: List[Optional[ElasticBuffer]] = [None] * num_ranks
        self.buffers: List[ElasticBuffer] = [ElasticBuffer(LocalGroup(self, r), **buffer_kwargs) for r in range(num_ranks)]
        self._C.Runtime.connect_local([b.runtime for b in self.buffers])
        _share_host_segments(self.buffers)
        torch.cuda.synchronize()

    def _register(self, rank: int, buffer) -> None:
        self._pending[rank] = buffer

    @property
    def runtimes(self):
        return [b.runtime for b in self.buffers]

    def barrier(self, with_cpu_sync: bool = True) -> None:
        self._C.Runtime.barrier(self.runtimes, True, with_cpu_sync)

    def dispatch(self, per_rank_kwargs: Sequence[dict]):
        """``per_rank_kwargs[r]`` holds the keyword arguments of ``ElasticBuffer.dispatch`` for rank r."""
        defaults = dict(topk_idx=None, topk_weights=None, cumulative_local_expert_recv_stats=None, num_experts=None,
                        num_max_tokens_per_rank=None, expert_alignment=None, num_sms=0, previous_event=None,
                        previous_event_before_epilogue=None, async_with_compute_stream=False,
                        allocate_on_comm_stream=False, handle=None, do_cpu_sync=None, do_expand=False,
                        do_zero_padding=False, use_tma_aligned_col_major_sf=False, zero_copy=False, fused_fp8=False,
                        round_scale=False, num_worst_tokens=0)
        args, metas = [], []
        for buf, kw in zip(self.buffers, per_rank_kwargs):
            kw = dict(kw)
            do_handle_copy = kw.pop('do_handle_copy', True)
            full = {**defaults, **kw}
            args.append(buf._make_dispatch_args(**full))
            metas.append((do_handle_copy, full['handle']))
        results = self._C.Runtime.dispatch(self.runtimes, args)
        return [buf._wrap_dispatch_result(r, a, copy, handle)
                for buf, r, a, (copy, handle) in zip(self.buffers, results, args, metas)]

    def combine(self, per_rank_kwargs: Sequence[dict]):
        defaults = dict(topk_weights=None, bias=None, num_sms=0, previous_event=None, previous_event_before_epilogue=None,
                        async_with_compute_stream=False, allocate_on_comm_stream=False, weighted=False)
        args = [buf._make_combine_args(**{**defaults, **kw}) for buf, kw in zip(self.buffers, per_rank_kwargs)]
        results = self._C.Runtime.combine(self.runtimes, args)
        return [(r.combined_x, r.combined_topk_weights, EventOverlap(r.event)) for r in results]

    # ------------------------------------------------------------------ low-latency mode
    def low_latency_dispatch(self, xs, topk_idxs, num_max_dispatch_tokens_per_rank: int, num_experts: int, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, phases: Optional[int] = None, ios=None,
                             num_sms: int = 0, shrink: bool = False):
        """All ranks' ``Buffer.low_latency_dispatch`` as one launch. Returns the per-rank IO blocks
        (``packed_recv_x``, ``packed_recv_sf``, ``packed_recv_count``, ``src_info``, ``layout_range``)."""
        C = self._C
        if ios is None:
            ios = []
            for x, idx in zip(xs, topk_idxs):
                io = C.LLDispatchIO()
                io.x, io.topk_idx = x, idx
                ios.append(io)
        phases = (C.LL_SEND | C.LL_RECV) if phases is None else phases
        C.ll_dispatch(self.runtimes, ios, num_max_dispatch_tokens_per_rank, num_experts, use_fp8, round_scale, use_ue8m0, phases,
                      num_sms, shrink, False, True)
        return ios

    def low_latency_combine(self, ys, topk_idxs, topk_weights, dispatch_ios, num_max_dispatch_tokens_per_rank: int,
                            num_experts: int, phases: Optional[int] = None, ios=None, num_sms: int = 0, shrink: bool = False,
                            use_logfmt: bool = False):
        C = self._C
        if ios is None:
            ios = []
            for y, idx, w, d in zip(ys, topk_idxs, topk_weights, dispatch_ios):
                io = C.LLCombineIO()
                io.x, io.topk_idx, io.topk_weights = y, idx, w
                io.src_info, io.layout_range = d.src_info, d.layout_range
                io.use_logfmt = use_logfmt
                ios.append(io)
        phases = (C.LL_SEND | C.LL_RECV) if phases is None else phases
        C.ll_combine(self.runtimes, ios, num_max_dispatch_tokens_per_rank, num_experts, phases, num_sms, shrink, False, True)
        return ios

    def check_status(self) -> None:
        for b in self.buffers:
            b.check_status()

    def destroy(self) -> None:
        torch.cuda.synchronize()
        for b in self.buffers:
            b.destroy()


class SingleProcessGroup:
    """A group of one rank for single-GPU use without ``torch.distributed`` (EP1)."""

    is_local_emulation = False

    def rank(self) -> int:
        return 0

    def size(self) -> int:
        return 1


class VirtualRanks:
    """Bare set of virtual ranks for subsystems that build their own buffers (tensor-parallel contexts,
    AGRS / PP sessions): hand ``groups[r]`` to the constructor of rank r's object, then call
    :meth:`connect` with the created buffers to wire their peer tables."""

    def __init__(self, num_ranks: int):
        self._C = require_native()
        self.num_ranks = num_ranks
        self.groups = [LocalGroup(self, r) for r in range(num_ranks)]
        self._registered = {}

    def _register(self, rank: int, buffer) -> None:
        self._registered[rank] = buffer

    def connect(self) -> None:
        buffers = [self._registered[r] for r in range(self.num_ranks)]
        self._C.Runtime.connect_local([b.runtime for b in buffers])
        _share_host_segments(buffers)
        torch.cuda.synchronize()
