"""``ElasticBuffer`` / ``EPHandle``: the high-throughput expert-parallel front end.

One ``ElasticBuffer`` per process (= per GPU) owns a symmetric heap that every peer of the
NVLink / NVSwitch domain maps, and drives the sm_100a dispatch / combine kernels that move
tokens with in-kernel peer stores. The Python surface (constructor keywords, ``dispatch`` and
``combine`` signatures and return tuples, size hints, SM model, barrier, AGRS / PP / Engram
entry points) follows deep_ep/buffers/elastic.py:25-1107 of the reference; keywords that
only make sense with an RDMA tier (``sl_idx``, ``num_allocated_qps``, ``num_qps``,
``allow_hybrid_mode``) are accepted and ignored.

Differences a caller can see:

* received rows are always in (source rank, token) order, so ``deterministic`` costs nothing;
* ``dispatch(x_bf16, ..., use_fp8_dispatch / fused_fp8=True)`` can cast to e4m3 with 1x128
  scales inside the dispatch kernel (the reference takes pre-quantised tuples only; those
  work here too);
* ``dispatch(..., zero_copy=True)`` returns ``recv_x`` (and row-major ``recv_sf``) as strided views of
  the receive region (valid until the second next dispatch on any rank of the group overwrites that half
  of the region) and skips the payload copy of the epilogue;
* ``combine(..., weighted=True)`` multiplies expanded rows by their top-k weights before summing;
* ``topk_idx`` may be int64 or int32 (``deepep_b200.topk_idx_t`` follows ``EP_NUM_TOPK_IDX_BITS``);
* device waits never trap: a wait that runs out records a status that :meth:`check_status`
  turns into :class:`EPTimeoutError`.
"""
from __future__ import annotations

import math
import os
from typing import Any, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist

from .._native import _C, require_native
from ..utils.envs import (check_nvlink_connections, check_torch_deterministic, get_logical_domain_size, get_nvlink_gbs,
                          get_physical_domain_size)
from ..utils.event import EventOverlap
from ..utils.math import align, ceil_div
from ..utils.semantic import value_or, weak_lru

QUANT_NONE, QUANT_E4M3, QUANT_E4M3_POW2 = 0, 1, 2


class EPHandle:
    """Routing metadata returned by :meth:`ElasticBuffer.dispatch`.

    It is consumed by :meth:`ElasticBuffer.combine` to send results back, and can be passed to a
    later ``dispatch(handle=...)`` to replay the same routing without counting or CPU sync.

    Attributes:
        do_expand: whether the expanded (one row per token and local expert) layout is used.
        num_experts, expert_alignment, num_max_tokens_per_rank, num_sms: settings of the dispatch.
        topk_idx: the routing ``[num_tokens, num_topk]`` (a clone unless ``do_handle_copy=False``).
        psum_num_recv_tokens_per_scaleup_rank: inclusive prefix sum of received tokens per source rank.
        psum_num_recv_tokens_per_expert: per local expert; non-expand: inclusive prefix of the aligned
            counts; expand: aligned start of the expert plus its real count.
        num_unaligned_recv_tokens_per_expert: real (token, expert) pair count per local expert.
        num_recv_tokens_per_expert_list: aligned counts as a Python list (only with CPU sync).
        recv_src_metadata: ``[num_recv_tokens, num_topk + 2]`` int32:
            ``{src_rank * num_max_tokens_per_rank + src_token, src_rank * num_topk + first local lane,
            expanded row per top-k lane or -1}``.
        dst_buffer_slot_idx: ``[num_tokens, num_ranks]`` row of each token in every destination
            rank's receive region (-1 = not sent there).
        dst_expanded_row_idx: ``[num_tokens, num_topk]`` row of each (token, expert) pair in the
            destination's expanded layout.
        num_recv_tokens / num_expanded_tokens: exact with CPU sync, else the worst case.
    """

    def __init__(self, do_expand: bool, num_experts: int, expert_alignment: int, num_max_tokens_per_rank: int,
                 num_sms: int, topk_idx: torch.Tensor, num_recv_tokens: int, num_expanded_tokens: int,
                 num_recv_tokens_per_expert_list: list, psum_num_recv_tokens_per_scaleup_rank: torch.Tensor,
                 psum_num_recv_tokens_per_expert: torch.Tensor, num_unaligned_recv_tokens_per_expert: torch.Tensor,
                 recv_src_metadata: torch.Tensor, dst_buffer_slot_idx: torch.Tensor,
                 dst_expanded_row_idx: Optional[torch.Tensor] = None,
                 token_metadata_at_forward: Optional[torch.Tensor] = None,
                 channel_linked_list: Optional[torch.Tensor] = None):
        assert topk_idx is not None
        self.do_expand = do_expand
        self.num_experts = num_experts
        self.expert_alignment = expert_alignment
        self.num_max_tokens_per_rank = num_max_tokens_per_rank
        self.num_sms = num_sms
        self.topk_idx = topk_idx
        self.num_recv_tokens = num_recv_tokens
        self.num_expanded_tokens = num_expanded_tokens
        self.num_recv_tokens_per_expert_list = num_recv_tokens_per_expert_list
        self.psum_num_recv_tokens_per_scaleup_rank = psum_num_recv_tokens_per_scaleup_rank
        self.psum_num_recv_tokens_per_expert = psum_num_recv_tokens_per_expert
        self.num_unaligned_recv_tokens_per_expert = num_unaligned_recv_tokens_per_expert
        self.recv_src_metadata = recv_src_metadata
        self.dst_buffer_slot_idx = dst_buffer_slot_idx
        self.dst_expanded_row_idx = dst_expanded_row_idx
        # single tier: the hybrid-mode members of the reference handle stay empty
        self.token_metadata_at_forward = token_metadata_at_forward
        self.channel_linked_list = channel_linked_list
        self._psum_expert_full: Optional[torch.Tensor] = None   # [local experts + 1], last = expanded rows
        # [ranks, ranks] tokens that rank i sent to rank j in this dispatch (every rank gets the whole matrix)
        self.num_tokens_per_rank_matrix: Optional[torch.Tensor] = None

    def deterministic_sort(self, *tensors):
        """Rows already arrive in (source rank, token) order; returns the tensors unchanged."""
        return tensors if len(tensors) != 1 else tensors[0]


class ElasticBuffer:
    """Expert-parallel communication buffer for one NVLink / NVSwitch domain.

    Supports high-throughput dispatch and combine, a GPU barrier, all-gather / reduce-scatter
    sessions (AGRS), pipeline send / recv (PP) and Engram table fetches.

    Attributes:
        group, rank_idx, num_ranks: the communication group and this rank's place in it.
        num_bytes: size of the symmetric heap (control area included).
        num_max_tokens_per_rank: default per-rank token bound.
        runtime: the native per-rank runtime.
    """

    def __init__(self, group: Any, num_bytes: Optional[int] = None, num_cpu_bytes: int = 0,
                 num_max_tokens_per_rank: int = 0, hidden: int = 0, num_topk: int = 0, use_fp8_dispatch: bool = False,
                 deterministic: bool = False, allow_hybrid_mode: bool = True, allow_multiple_reduction: bool = True,
                 prefer_overlap_with_compute: bool = True, sl_idx: int = 3, num_allocated_qps: int = 0,
                 num_cpu_timeout_secs: float = 300, num_gpu_timeout_secs: float = 100, explicitly_destroy: bool = False):
        require_native()
        self.group = group
        self.rank_idx = group.rank()
        self.num_ranks = group.size()
        assert 1 <= self.num_ranks <= _C.MAX_RANKS, f'one NVLink domain holds at most {_C.MAX_RANKS} ranks'
        self.allow_hybrid_mode = allow_hybrid_mode
        self.allow_multiple_reduction = allow_multiple_reduction
        # How the combine's reduce overlaps the sends (EP_COMBINE_FUSED_REDUCE): 1 (default) = a reduce kernel runs
        # beside the send kernel on the SMs it leaves free and sums a token as soon as all its rows have been counted
        # as landed; 0 = the reduce kernel runs after the send kernel.
        self.fuse_combine_reduce = int(os.environ.get('EP_COMBINE_FUSED_REDUCE', '1'))
        self.prefer_overlap_with_compute = prefer_overlap_with_compute
        self.deterministic = deterministic
        self.use_fp8_dispatch = use_fp8_dispatch
        self.explicitly_destroy = explicitly_destroy
        self.num_allocated_qps = num_allocated_qps
        self.num_cpu_bytes = num_cpu_bytes

        if num_bytes is None:
            assert num_max_tokens_per_rank > 0 and hidden > 0, 'give num_bytes or the MoE settings'
            num_bytes = self.get_buffer_size_hint(group, num_max_tokens_per_rank, hidden, max(num_topk, 1), use_fp8_dispatch)
        assert num_bytes % self.get_elastic_buffer_alignment() == 0
        num_bytes = max(int(num_bytes), int(_C.CONTROL_BYTES) + self.get_elastic_buffer_alignment())
        if os.environ.get('EP_BUFFER_DEBUG'):
            print(f'EP elastic buffer: {num_bytes} bytes at rank {self.rank_idx}/{self.num_ranks}', flush=True)
        self.num_bytes = num_bytes
        self.num_max_tokens_per_rank = num_max_tokens_per_rank

        # EP_HEAP_BACKEND=vmm: the heap comes from CUDA's virtual memory management and the CPU segment, if any, sits
        # in the same address range right behind the GPU segment; default: cudaMalloc + CUDA IPC, CPU segment apart
        self.heap_is_vmm = bool(_C.Runtime.heap_backend_is_vmm())
        self.runtime = _C.Runtime(self.rank_idx, self.num_ranks, num_bytes, float(num_gpu_timeout_secs),
                                  float(num_cpu_timeout_secs), num_cpu_bytes if self.heap_is_vmm else 0)
        self._destroyed = False
        if not self.heap_is_vmm:
            self._connect_host_segments()
        self._connect()
        if self.heap_is_vmm:
            self.host_segments = []
            if num_cpu_bytes > 0:
                # (the emulated cluster completes the list once all virtual ranks exist)
                ranks = [self.rank_idx] if getattr(self.group, 'is_local_emulation', False) else range(self.num_ranks)
                self.host_segments = [_C.HostSegment.window(self.runtime, r) for r in ranks]

        self.num_scaleout_ranks, self.num_scaleup_ranks = self.get_logical_domain_size()
        self.scaleout_rank_idx = self.rank_idx // self.num_scaleup_ranks
        self.scaleup_rank_idx = self.rank_idx % self.num_scaleup_ranks
        self.num_rdma_ranks, self.num_nvlink_ranks = self.get_physical_domain_size()
        self._pp = None
        self._agrs = None
        self._engram = None

    # ------------------------------------------------------------------ set-up / tear-down
    def _connect(self) -> None:
        """Exchanges the heap handles over the group and maps every peer's heap."""
        if getattr(self.group, 'is_local_emulation', False):
            self.group.register(self)      # the emulated cluster wires the peers once all ranks exist
            return
        if self.num_ranks > 1:
            check_nvlink_connections(self.group)
            handles: List[Optional[bytes]] = [None] * self.num_ranks
            dist.all_gather_object(handles, self.runtime.export_handle(), group=self.group)
            self.runtime.open_peers(handles)
        torch.cuda.synchronize()
        if self.num_ranks > 1:
            dist.barrier(group=self.group)
            self.runtime.finish_export()       # every peer has mapped this rank's heap: stop handing out descriptors
        torch.cuda.synchronize()

    def _connect_host_segments(self) -> None:
        """``num_cpu_bytes > 0``: one pinned host segment per rank (POSIX shared memory registered with CUDA), mapped
        by every rank of the machine. ``host_segments[r]`` is rank r's segment as this process addresses it."""
        self.host_segments = []
        if self.num_cpu_bytes <= 0:
            return
        own = _C.HostSegment.create(self.num_cpu_bytes)
        if getattr(self.group, 'is_local_emulation', False):
            self.host_segments = [own]          # completed by the emulated cluster once all ranks exist
            return
        names: List[Optional[str]] = [None] * self.num_ranks
        if self.num_ranks > 1:
            dist.all_gather_object(names, own.name, group=self.group)
        self.host_segments = [own if r == self.rank_idx else _C.HostSegment.open(names[r], self.num_cpu_bytes)
                              for r in range(self.num_ranks)]
        if self.num_ranks > 1:
            dist.barrier(group=self.group)     # everybody has opened every name before an owner may unlink it

    def destroy(self) -> None:
        """Releases the heap. Collective when ``explicitly_destroy`` was set (peers unmap first)."""
        if self._destroyed:
            return
        self._destroyed = True
        torch.cuda.synchronize()
        if self.num_ranks > 1 and not getattr(self.group, 'is_local_emulation', False) and self.explicitly_destroy:
            dist.barrier(group=self.group)
        for seg in getattr(self, 'host_segments', []):
            seg.release()
        self.host_segments = []
        self.runtime.destroy()

    def __del__(self):
        try:
            if not getattr(self, '_destroyed', True) and not self.explicitly_destroy:
                self._destroyed = True
                self.runtime.destroy()
        except Exception:   # interpreter shutdown
            pass

    def check_status(self) -> None:
        """Raises :class:`EPTimeoutError` if a bounded device wait of this rank has run out."""
        self.runtime.check_status()

    # ------------------------------------------------------------------ size hints
    @staticmethod
    def get_elastic_buffer_alignment() -> int:
        return int(_C.HEAP_ALIGNMENT) if _C is not None else 2 << 20

    @staticmethod
    def get_buffer_size_hint(group: Any, num_max_tokens_per_rank: int, hidden: int, num_topk: int = 0,
                             use_fp8_dispatch: bool = False, allow_hybrid_mode: bool = True,
                             allow_multiple_reduction: bool = True) -> int:
        """Heap bytes for EP with these settings: control area, two dispatch receive regions sized for
        bf16 rows (an FP8 dispatch fits as well) and two combine regions."""
        require_native()
        return int(_C.Runtime.ht_buffer_size(group.size(), num_max_tokens_per_rank, hidden, max(num_topk, 1)))

    @staticmethod
    def get_engram_storage_size_hint(num_entries: int, hidden: int, dtype: torch.dtype = torch.bfloat16,
                                     num_ranks: int = 1) -> int:
        """Heap bytes for this rank's shard of an Engram table (entries split evenly over the ranks)."""
        per_rank = ceil_div(num_entries, num_ranks)
        elem = torch.empty(0, dtype=dtype).element_size()
        return align(int(_C.CONTROL_BYTES) + per_rank * hidden * elem, ElasticBuffer.get_elastic_buffer_alignment())

    @staticmethod
    def get_pp_buffer_size_hint(num_max_tensor_bytes: int, num_max_inflight_tensors: int) -> int:
        """Heap bytes for the PP slot rings (one ring per direction)."""
        slot = align(num_max_tensor_bytes, 256)
        return align(int(_C.CONTROL_BYTES) + 2 * num_max_inflight_tensors * slot, ElasticBuffer.get_elastic_buffer_alignment())

    @staticmethod
    def get_agrs_num_max_session_bytes(group: Any, num_bytes: int) -> int:
        """Largest per-rank session payload that a heap of ``num_bytes`` can gather."""
        usable = num_bytes - int(_C.CONTROL_BYTES)
        return max(0, usable // group.size() // 256 * 256)

    @staticmethod
    def get_agrs_buffer_size_hint(group: Any, num_max_session_bytes: int) -> int:
        """Heap bytes for all-gather sessions of up to ``num_max_session_bytes`` per rank."""
        return align(int(_C.CONTROL_BYTES) + group.size() * align(num_max_session_bytes, 256),
                     ElasticBuffer.get_elastic_buffer_alignment())

    # ------------------------------------------------------------------ misc API
    def barrier(self, use_comm_stream: bool = True, with_cpu_sync: bool = False, sequential: bool = True) -> None:
        """GPU barrier over the group (bounded wait; ``with_cpu_sync`` also waits on the host)."""
        _C.Runtime.barrier([self.runtime], use_comm_stream, with_cpu_sync)

    @staticmethod
    def capture():
        """An event recorded on the current stream (to be passed as ``previous_event``)."""
        require_native()
        return _C.EventHandle()

    def get_comm_stream(self) -> torch.cuda.Stream:
        stream_id, device_index, device_type = self.runtime.comm_stream_id()
        return torch.cuda.Stream(stream_id=stream_id, device_index=device_index, device_type=device_type)

    def get_physical_domain_size(self) -> Tuple[int, int]:
        return get_physical_domain_size(self.group)

    def get_logical_domain_size(self) -> Tuple[int, int]:
        return get_logical_domain_size(self.group, self.allow_hybrid_mode)

    # ------------------------------------------------------------------ Engram / PP / AGRS (experimental in the reference too)
    def _engram_store(self):
        if self._engram is None:
            from ..parallel.engram import EngramStore
            self._engram = EngramStore(self)
        return self._engram

    def engram_write(self, storage: torch.Tensor, sf: Optional[torch.Tensor] = None) -> None:
        """Stores this rank's shard ``[entries_per_rank, hidden]`` (bf16, or e4m3 with the replicated scale
        table ``sf [total entries, packs]``) in the heap. Barriers before and after."""
        self._engram_store().write(storage, sf)

    def engram_fetch(self, indices: torch.Tensor, num_qps: int = 0, use_tma_aligned_col_major_sf: bool = False):
        """Starts fetching the rows ``indices [tokens, entries per token]`` (int32) from their owner ranks and
        returns a hook; ``hook()`` waits and returns ``(data [tokens * entries, hidden], sf or None)``."""
        return self._engram_store().fetch(indices, use_tma_aligned_col_major_sf)

    def _pp_ring(self):
        if self._pp is None:
            from ..parallel.pp import PipelineRing
            self._pp = PipelineRing(self)
        return self._pp

    def pp_set_config(self, num_max_tensor_bytes: int, num_max_inflight_tensors: int):
        """Sizes the PP slot rings. Includes a barrier to flush earlier operations on the heap."""
        self.barrier()
        self._pp_ring().set_config(num_max_tensor_bytes, num_max_inflight_tensors)
        self.barrier()

    def pp_send(self, t: torch.Tensor, dst_rank_idx: int, num_sms: int = 0) -> None:
        """Sends ``t`` to the previous or next rank of the ring (copy engine, no SMs)."""
        self._pp_ring().send(t, dst_rank_idx)

    def pp_recv(self, t: torch.Tensor, src_rank_idx: int, num_sms: int = 0) -> None:
        """Receives into ``t`` from the previous or next rank of the ring."""
        self._pp_ring().recv(t, src_rank_idx)

    def _agrs_manager(self):
        if self._agrs is None:
            from ..parallel.agrs import AgrsManager
            self._agrs = AgrsManager(self)
        return self._agrs

    def create_agrs_session(self) -> None:
        self._agrs_manager().create_session()

    def destroy_agrs_session(self) -> None:
        self._agrs_manager().destroy_session()

    def agrs_new_session(self, enabled: bool = True):
        """Context manager around :meth:`create_agrs_session` / :meth:`destroy_agrs_session`."""
        from contextlib import contextmanager

        @contextmanager
        def session():
            if not enabled:
                yield
                return
            self.create_agrs_session()
            try:
                yield
            finally:
                self.destroy_agrs_session()
        return session()

    def agrs_set_config(self, num_max_session_bytes: int, num_max_all_gathers_per_session: int) -> None:
        self.barrier()
        self._agrs_manager().set_config(num_max_session_bytes, num_max_all_gathers_per_session)
        self.barrier()

    def agrs_get_inplace_tensor(self, shapes, dtype: torch.dtype):
        """Tensor(s) inside this rank's slot of the next all-gather(s) of the open session."""
        return self._agrs_manager().get_inplace_tensor(shapes, dtype)

    def all_gather(self, t: Union[torch.Tensor, Sequence[torch.Tensor]]):
        """All-gather inside the open AGRS session: returns ``(gathered [ranks, ...], handle)`` (or
        ``(*gathered, handle)`` for a sequence); ``handle()`` makes the current stream wait for arrival."""
        return self._agrs_manager().all_gather(t)

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """Sum over ranks of ``t`` (bf16 / fp32, leading dim divisible by the ranks), scattered by leading chunk."""
        return self._agrs_manager().reduce_scatter(t)

    # ------------------------------------------------------------------ SM / QP model
    @weak_lru(maxsize=None)
    def get_theoretical_num_sms(self, num_experts: int, num_topk: int, num_scaleout_topk: int = 0, rdma_gbs: float = 0,
                                nvlink_gbs: float = 0, sm_read_gbs: float = 200, sm_write_gbs: float = 50) -> int:
        """SM count at which the dispatch / combine kernels stop being SM-bound (balanced gate).

        Per received row a sending SM reads ``1 / d`` rows (``d`` = expected number of distinct
        destination ranks of a token, each row is loaded once and stored ``d`` times) and writes
        one row; ``(R - 1) / R`` of the rows cross NVLink. The SM count is the larger of
        ``nvlink / traffic * read / sm_read`` and ``nvlink / traffic * write / sm_write``, with 25 %
        head-room, rounded up to an even number of at least 4; without ``prefer_overlap_with_compute``
        at least 64 SMs are used. EP8 / 256 experts / top-8 with 810 GB/s gives 24.
        """
        assert num_scaleout_topk == 0
        num_device_sms = torch.cuda.get_device_properties('cuda').multi_processor_count if torch.cuda.is_available() else 148
        ranks = self.num_ranks
        if ranks == 1:
            return num_device_sms
        nvlink_gbs = nvlink_gbs or get_nvlink_gbs()
        miss = math.comb(num_experts - num_experts // ranks, num_topk) / math.comb(num_experts, num_topk)
        expected_ranks = ranks * (1 - miss)
        read, write = 1 / expected_ranks, 1.0
        traffic = 1 - 1 / ranks
        need = max(nvlink_gbs / traffic * read / sm_read_gbs, nvlink_gbs / traffic * write / sm_write_gbs)
        num_sms = align(max(4, math.ceil(need * 1.25)), 2)
        if not self.prefer_overlap_with_compute:
            num_sms = max(num_sms, 64)
        num_sms = min(num_sms, num_device_sms)
        if os.environ.get('EP_BUFFER_DEBUG'):
            print(f'EP SM model: {expected_ranks=:.3f} {read=:.3f} {write=} {traffic=:.3f} {nvlink_gbs=} {num_sms=}', flush=True)
        return num_sms

    def get_theoretical_num_qps(self, num_sms: int) -> int:
        """No RDMA tier: there are no queue pairs to size."""
        return 0

    # ------------------------------------------------------------------ dispatch
    def _make_dispatch_args(self, x, topk_idx, topk_weights, cumulative_local_expert_recv_stats, num_experts,
                            num_max_tokens_per_rank, expert_alignment, num_sms, previous_event,
                            previous_event_before_epilogue, async_with_compute_stream, allocate_on_comm_stream, handle,
                            do_cpu_sync, do_expand, do_zero_padding, use_tma_aligned_col_major_sf, zero_copy, fused_fp8,
                            round_scale, num_worst_tokens=0):
        a = _C.DispatchArgs()
        if isinstance(x, tuple):
            a.x, a.sf = x
            assert not fused_fp8, 'fused FP8 casting takes a bf16 tensor, not a pre-quantised tuple'
        else:
            a.x = x
        if handle is not None:
            assert topk_idx is None, '`topk_idx` is taken from the handle'
            assert cumulative_local_expert_recv_stats is None
            num_experts = value_or(num_experts, handle.num_experts)
            num_max_tokens_per_rank = value_or(num_max_tokens_per_rank, handle.num_max_tokens_per_rank)
            expert_alignment = value_or(expert_alignment, handle.expert_alignment)
            assert num_experts == handle.num_experts and num_max_tokens_per_rank == handle.num_max_tokens_per_rank
            assert expert_alignment == handle.expert_alignment and do_expand == handle.do_expand
            topk_idx = handle.topk_idx
            a.cached = True
            a.h_token_slot = handle.dst_buffer_slot_idx
            a.h_pair_row = handle.dst_expanded_row_idx
            a.h_psum_rank = handle.psum_num_recv_tokens_per_scaleup_rank
            a.h_psum_expert = handle._psum_expert_full
            a.h_num_unaligned = handle.num_unaligned_recv_tokens_per_expert
            a.h_recv_src_metadata = handle.recv_src_metadata
            a.h_num_recv_tokens = handle.num_recv_tokens
            a.h_num_expanded_tokens = handle.num_expanded_tokens
            do_cpu_sync = False
        assert num_experts is not None and topk_idx is not None
        num_max_tokens_per_rank = value_or(num_max_tokens_per_rank, self.num_max_tokens_per_rank)
        assert num_max_tokens_per_rank > 0, 'num_max_tokens_per_rank is unknown'
        a.topk_idx = topk_idx
        a.topk_weights = topk_weights
        a.cumulative_stats = cumulative_local_expert_recv_stats
        a.num_experts = num_experts
        a.num_max_tokens = num_max_tokens_per_rank
        a.expert_alignment = value_or(expert_alignment, 1)
        a.num_sms = num_sms if num_sms > 0 else self.get_theoretical_num_sms(num_experts, topk_idx.size(1))
        a.quant_mode = (QUANT_E4M3_POW2 if round_scale else QUANT_E4M3) if fused_fp8 else QUANT_NONE
        a.do_expand = do_expand
        a.do_zero_padding = do_zero_padding
        a.do_cpu_sync = value_or(do_cpu_sync, True)
        a.zero_copy = zero_copy
        a.num_worst_tokens = num_worst_tokens
        a.col_major_sf = use_tma_aligned_col_major_sf
        sc = a.sc
        sc.previous_event = previous_event
        sc.previous_event_before_epilogue = previous_event_before_epilogue
        sc.async_with_compute_stream = async_with_compute_stream
        sc.allocate_on_comm_stream = allocate_on_comm_stream
        a.sc = sc
        return a

    def _wrap_dispatch_result(self, r, a, do_handle_copy: bool, handle: Optional[EPHandle]):
        num_local = a.num_experts // self.num_ranks
        if handle is None:
            topk_idx = a.topk_idx.clone() if do_handle_copy else a.topk_idx
            new_handle = EPHandle(a.do_expand, a.num_experts, a.expert_alignment, a.num_max_tokens, r.num_sms, topk_idx,
                                  r.num_recv_tokens, r.num_expanded_tokens, r.num_recv_tokens_per_expert_list,
                                  r.psum_rank, r.psum_expert[:num_local], r.num_unaligned, r.recv_src_metadata,
                                  r.token_slot, r.pair_row)
            new_handle._psum_expert_full = r.psum_expert
            new_handle.num_tokens_per_rank_matrix = r.count_matrix
        else:
            new_handle = handle
        recv_x = (r.recv_x, r.recv_sf) if r.recv_sf is not None else r.recv_x
        return recv_x, r.recv_topk_idx, r.recv_topk_weights, new_handle, EventOverlap(r.event)

    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], topk_idx: Optional[torch.Tensor] = None,
                 topk_weights: Optional[torch.Tensor] = None,
                 cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None, num_experts: Optional[int] = None,
                 num_max_tokens_per_rank: Optional[int] = None, expert_alignment: Optional[int] = None, num_sms: int = 0,
                 num_qps: int = 0, previous_event=None, previous_event_before_epilogue=None,
                 async_with_compute_stream: bool = False, allocate_on_comm_stream: bool = False,
                 handle: Optional[EPHandle] = None, do_handle_copy: bool = True, do_cpu_sync: Optional[bool] = None,
                 do_expand: bool = False, do_zero_padding: bool = False, use_tma_aligned_col_major_sf: bool = False,
                 zero_copy: bool = False, fused_fp8: Optional[bool] = None, round_scale: bool = False,
                 num_worst_tokens: int = 0):
        """Sends every token to the ranks that own its selected experts.

        Arguments follow the reference (deep_ep/buffers/elastic.py:855-923): ``x`` is bf16
        ``[tokens, hidden]`` or an ``(e4m3, scales)`` tuple; ``topk_idx`` int64 ``[tokens, topk]`` with
        -1 for unused lanes; ``handle`` replays an earlier routing. Extras: ``fused_fp8`` casts a bf16
        ``x`` to e4m3 with 1x128 float scales inside the kernel (default: on when the buffer was built
        with ``use_fp8_dispatch`` and ``x`` is bf16); ``round_scale`` makes those scales powers of two;
        ``zero_copy`` returns ``recv_x`` (and row-major scales) as strided views of the receive region: they stay
        valid until the second next dispatch of any rank of the group, which overwrites that half of the region;
        ``num_worst_tokens`` (with ``do_cpu_sync=False``) sets the row count of the outputs, whose routing rows
        past the received count are filled with -1 / 0.

        Returns ``(recv_x | (recv_x, recv_sf), recv_topk_idx, recv_topk_weights, handle, event)``.
        In the expanded layout ``recv_topk_idx`` is ``None`` and ``recv_topk_weights`` is 1-D.
        """
        check_torch_deterministic()
        if fused_fp8 is None:
            fused_fp8 = self.use_fp8_dispatch and not isinstance(x, tuple) and x.dtype == torch.bfloat16
        a = self._make_dispatch_args(x, topk_idx, topk_weights, cumulative_local_expert_recv_stats, num_experts,
                                     num_max_tokens_per_rank, expert_alignment, num_sms, previous_event,
                                     previous_event_before_epilogue, async_with_compute_stream, allocate_on_comm_stream,
                                     handle, do_cpu_sync, do_expand, do_zero_padding, use_tma_aligned_col_major_sf,
                                     zero_copy, fused_fp8, round_scale, num_worst_tokens)
        r = _C.Runtime.dispatch([self.runtime], [a])[0]
        return self._wrap_dispatch_result(r, a, do_handle_copy, handle)

    # ------------------------------------------------------------------ combine
    @staticmethod
    def _unpack_bias(bias) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        if bias is None:
            return None, None
        if isinstance(bias, torch.Tensor):
            return bias, None
        assert len(bias) == 2
        return bias[0], bias[1]

    def _make_combine_args(self, x, handle, topk_weights, bias, num_sms, previous_event, previous_event_before_epilogue,
                           async_with_compute_stream, allocate_on_comm_stream, weighted=False):
        a = _C.CombineArgs()
        a.x = x
        a.topk_weights = topk_weights
        a.bias0, a.bias1 = self._unpack_bias(bias)
        a.recv_src_metadata = handle.recv_src_metadata
        a.topk_idx = handle.topk_idx
        a.psum_rank = handle.psum_num_recv_tokens_per_scaleup_rank
        a.num_experts = handle.num_experts
        a.num_max_tokens = handle.num_max_tokens_per_rank
        a.num_sms = num_sms if num_sms > 0 else handle.num_sms
        a.do_expand = handle.do_expand
        a.weighted = bool(weighted)
        a.allow_multiple_reduction = self.allow_multiple_reduction
        a.dst_slot = handle.dst_buffer_slot_idx
        a.count_matrix = handle.num_tokens_per_rank_matrix
        a.fuse_reduce = self.fuse_combine_reduce
        sc = a.sc
        sc.previous_event = previous_event
        sc.previous_event_before_epilogue = previous_event_before_epilogue
        sc.async_with_compute_stream = async_with_compute_stream
        sc.allocate_on_comm_stream = allocate_on_comm_stream
        a.sc = sc
        return a

    def combine(self, x: torch.Tensor, handle: EPHandle, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[None, torch.Tensor, Tuple[torch.Tensor, torch.Tensor]] = None, num_sms: int = 0,
                num_qps: int = 0, previous_event=None, previous_event_before_epilogue=None,
                async_with_compute_stream: bool = False, allocate_on_comm_stream: bool = False, weighted: bool = False):
        """Sends expert outputs back to the tokens' source ranks and sums them there.

        ``x`` is bf16: one row per received token (non-expand; the caller has summed its local
        experts) or one row per expanded row. The result is the plain sum of all contributions plus
        ``bias`` (fp32 accumulation in ascending rank order, one bf16 rounding at the end; with the
        expanded layout and ``allow_multiple_reduction`` each rank's partial sum is rounded once
        more). ``topk_weights`` are carried back to ``combined_topk_weights``; with ``weighted=True`` (expanded
        layout only) every expanded row is also multiplied by its weight before it is added, i.e. the result is
        ``sum_k w_k * x_k`` as the low-latency combine computes it.

        Returns ``(combined_x, combined_topk_weights, event)``.
        """
        check_torch_deterministic()
        a = self._make_combine_args(x, handle, topk_weights, bias, num_sms, previous_event, previous_event_before_epilogue,
                                    async_with_compute_stream, allocate_on_comm_stream, weighted)
        r = _C.Runtime.combine([self.runtime], [a])[0]
        return r.combined_x, r.combined_topk_weights, EventOverlap(r.event)
