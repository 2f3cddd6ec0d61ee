"""``Buffer`` / ``Config``: the first-generation front end (layout query, normal dispatch / combine,
low-latency dispatch / combine with receive hooks, rank masking).

The call signatures and return tuples follow deep_ep/buffers/legacy.py:14-713 of the reference so
that code written against it keeps working. Underneath there is one NVLink tier and one set of
kernels: the normal mode drives the same high-throughput dispatch / combine kernels as
``ElasticBuffer`` (so rows arrive in (source rank, token) order and no chunk-size tuning exists:
``Config`` only carries the SM count), the low-latency mode drives the ``ll`` kernels.
Arguments that only make sense with RDMA (``num_qps_per_rank``, ``allow_mnnvl``, ``comm``,
``num_tokens_per_rdma_rank`` ...) are accepted and ignored.
"""
from __future__ import annotations

import contextlib

from typing import Any, Callable, List, Optional, Tuple, Union

import torch
import torch.distributed as dist

from .._native import _C, require_native
from ..utils.envs import check_torch_deterministic
from ..utils.event import EventOverlap
from .elastic import ElasticBuffer, EPHandle


class Config:
    """Tuning knobs of the normal-mode kernels. Only ``num_sms`` has an effect here; the chunk sizes of
    the reference's queue-based kernels are kept as attributes for compatibility."""

    def __init__(self, num_sms: int = 24, num_max_nvl_chunked_send_tokens: int = 6, num_max_nvl_chunked_recv_tokens: int = 256,
                 num_max_rdma_chunked_send_tokens: int = 6, num_max_rdma_chunked_recv_tokens: int = 256):
        self.num_sms = num_sms
        self.num_max_nvl_chunked_send_tokens = num_max_nvl_chunked_send_tokens
        self.num_max_nvl_chunked_recv_tokens = num_max_nvl_chunked_recv_tokens
        self.num_max_rdma_chunked_send_tokens = num_max_rdma_chunked_send_tokens
        self.num_max_rdma_chunked_recv_tokens = num_max_rdma_chunked_recv_tokens

    def get_nvl_buffer_size_hint(self, hidden_bytes: int, num_ranks: int, num_max_tokens_per_rank: int = 4096,
                                 num_topk: int = 8) -> int:
        """Heap bytes for normal mode with rows of ``hidden_bytes`` (bf16: 2 * hidden)."""
        require_native()
        return int(_C.Runtime.ht_buffer_size(num_ranks, num_max_tokens_per_rank, max(hidden_bytes // 2, 1), num_topk))

    def get_rdma_buffer_size_hint(self, hidden_bytes: int, num_ranks: int) -> int:
        """No RDMA tier."""
        return 0


class LegacyHandle(tuple):
    """The 6-tuple the reference returns from ``dispatch`` (``rank_prefix_matrix, channel_prefix_matrix,
    recv_channel_prefix_matrix, recv_src_idx, is_token_in_rank, send_head``) plus the native handle."""

    ep_handle: EPHandle

    def __new__(cls, items, ep_handle: EPHandle):
        obj = super().__new__(cls, items)
        obj.ep_handle = ep_handle
        return obj


class Buffer:
    """First-generation communication buffer (normal mode + low-latency mode) on one NVLink domain.

    Attributes:
        num_sms: SMs used by the normal-mode kernels (class-wide, see :meth:`set_num_sms`).
        rank, group_size, group: place in the communication group.
        num_nvl_bytes: heap bytes requested for normal mode.
        num_rdma_bytes: heap bytes requested for low-latency mode (the name is historical: the
            low-latency kernels use NVLink here).
    """

    num_sms: int = 24

    def __init__(self, group: Any, num_nvl_bytes: int = 0, num_rdma_bytes: int = 0, low_latency_mode: bool = False,
                 num_qps_per_rank: int = 24, allow_nvlink_for_low_latency_mode: bool = True, allow_mnnvl: bool = False,
                 explicitly_destroy: bool = False, enable_shrink: bool = False, comm: Any = None,
                 num_gpu_timeout_secs: float = 100, num_cpu_timeout_secs: float = 100) -> None:
        require_native()
        check_torch_deterministic()
        self.group = group
        self.rank = group.rank()
        self.group_size = group.size()
        self.num_nvl_bytes = num_nvl_bytes
        self.num_rdma_bytes = num_rdma_bytes
        self.low_latency_mode = low_latency_mode
        self.explicitly_destroy = explicitly_destroy
        self.enable_shrink = enable_shrink
        align = ElasticBuffer.get_elastic_buffer_alignment()
        num_bytes = max(num_nvl_bytes, num_rdma_bytes, int(_C.CONTROL_BYTES) + align)
        num_bytes = -(-num_bytes // align) * align
        # one heap serves both modes (their regions overlap: do not interleave the two modes without a barrier)
        self._elastic = ElasticBuffer(group, num_bytes=num_bytes, num_gpu_timeout_secs=num_gpu_timeout_secs,
                                      num_cpu_timeout_secs=num_cpu_timeout_secs, explicitly_destroy=explicitly_destroy)
        self.runtime = self._elastic.runtime
        self._tmax_cache = {}

    # ------------------------------------------------------------------ misc
    def destroy(self):
        self._elastic.destroy()

    def check_status(self) -> None:
        self.runtime.check_status()

    @staticmethod
    def is_sm90_compiled() -> bool:
        """The kernels are built for sm_100a only; kept for API compatibility."""
        return True

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        assert new_num_sms % 2 == 0, 'the SM count must be even'
        Buffer.num_sms = new_num_sms

    @staticmethod
    def capture() -> EventOverlap:
        return EventOverlap(_C.EventHandle())

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int, num_experts: int) -> int:
        """Heap bytes for low-latency mode (two halves of receive, combine and staging areas)."""
        require_native()
        return int(_C.ll_buffer_size(num_ranks, num_max_dispatch_tokens_per_rank, hidden, num_experts))

    def get_comm_stream(self) -> torch.cuda.Stream:
        return self._elastic.get_comm_stream()

    def get_local_buffer_tensor(self, dtype: torch.dtype, size: Optional[torch.Size] = None, offset: int = 0,
                                use_rdma_buffer: bool = False) -> torch.Tensor:
        """A view of this rank's heap (after the control area) as ``dtype``."""
        base = int(_C.CONTROL_BYTES) + offset
        raw = self.runtime.heap_tensor(base, self.runtime.num_bytes() - base)
        elem = torch.empty(0, dtype=dtype).element_size()
        t = raw[:raw.numel() // elem * elem].view(dtype)
        return t if size is None else t[:size.numel()].view(size)

    @staticmethod
    def get_dispatch_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    @staticmethod
    def get_combine_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    # ------------------------------------------------------------------ normal mode
    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event: Optional[EventOverlap] = None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """``(num_tokens_per_rank, None, num_tokens_per_expert, is_token_in_rank, event)`` for ``topk_idx``."""
        r = _C.get_dispatch_layout(self.runtime, topk_idx, num_experts, getattr(previous_event, 'event', None), async_finish,
                                   allocate_on_comm_stream)
        return r[0], None, r[1], r[2], EventOverlap(r[3])

    def _max_tokens(self, hidden: int, num_topk: int) -> int:
        """Largest per-rank token bound whose regions fit the heap (the same on every rank)."""
        key = (hidden, num_topk)
        if key not in self._tmax_cache:
            total, lo, hi = self.runtime.num_bytes(), 1, 1 << 20
            assert _C.Runtime.ht_buffer_size(self.group_size, lo, hidden, num_topk) <= total, 'buffer too small for this hidden size'
            while lo < hi:
                mid = (lo + hi + 1) // 2
                if _C.Runtime.ht_buffer_size(self.group_size, mid, hidden, num_topk) <= total:
                    lo = mid
                else:
                    hi = mid - 1
            self._tmax_cache[key] = lo
        return self._tmax_cache[key]

    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], handle: Optional[Tuple] = None,
                 num_tokens_per_rank: Optional[torch.Tensor] = None, num_tokens_per_rdma_rank: Optional[torch.Tensor] = None,
                 is_token_in_rank: Optional[torch.Tensor] = None, num_tokens_per_expert: Optional[torch.Tensor] = None,
                 topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None, expert_alignment: int = 1,
                 num_worst_tokens: int = 0, config: Optional[Config] = None, previous_event: Optional[EventOverlap] = None,
                 async_finish: bool = False, allocate_on_comm_stream: bool = False, num_experts: Optional[int] = None):
        """Normal-mode dispatch. Returns ``(recv_x, recv_topk_idx, recv_topk_weights,
        num_recv_tokens_per_expert_list, handle, event)``; with a cached ``handle`` only ``recv_x`` and the
        event are meaningful. ``num_worst_tokens > 0`` skips the CPU sync and returns worst-case shapes.
        ``num_experts`` is inferred from ``num_tokens_per_expert`` when not given."""
        config = config or self.get_dispatch_config(self.group_size)
        hidden = (x[0] if isinstance(x, tuple) else x).size(1)
        prev = getattr(previous_event, 'event', None)
        if handle is not None:
            assert topk_idx is None and topk_weights is None
            ep_handle = handle.ep_handle
            recv_x, _, _, _, event = self._elastic.dispatch(
                x, handle=ep_handle, num_sms=config.num_sms, previous_event=prev, async_with_compute_stream=async_finish,
                allocate_on_comm_stream=allocate_on_comm_stream)
            return recv_x, None, None, None, None, event
        assert topk_idx is not None, 'the routing (`topk_idx`) is needed to dispatch'
        if num_experts is None:
            assert num_tokens_per_expert is not None
            num_experts = num_tokens_per_expert.numel()
        t_max = self._max_tokens(hidden, topk_idx.size(1))
        # num_worst_tokens > 0: no CPU sync (graph-safe); the outputs have exactly that many rows and the routing
        # rows past the received count hold -1 / 0 (csrc/legacy/buffer.hpp:571-577, intranode.cu:536-540 of the reference)
        assert num_worst_tokens <= self.group_size * t_max, 'num_worst_tokens exceeds what the buffer can receive'
        recv_x, recv_topk_idx, recv_topk_weights, ep_handle, event = self._elastic.dispatch(
            x, topk_idx=topk_idx, topk_weights=topk_weights, num_experts=num_experts, num_max_tokens_per_rank=t_max,
            expert_alignment=expert_alignment, num_sms=config.num_sms, previous_event=prev,
            async_with_compute_stream=async_finish, allocate_on_comm_stream=allocate_on_comm_stream,
            do_cpu_sync=num_worst_tokens == 0, fused_fp8=False, num_worst_tokens=num_worst_tokens)
        if recv_topk_weights is not None:
            # weights of experts that live elsewhere carry no meaning on this rank
            if async_finish:
                with torch.cuda.stream(self.get_comm_stream()):
                    recv_topk_weights.masked_fill_(recv_topk_idx < 0, 0)
                    event = EventOverlap(_C.EventHandle())
            else:
                recv_topk_weights.masked_fill_(recv_topk_idx < 0, 0)
        if is_token_in_rank is None:
            is_token_in_rank = ep_handle.dst_buffer_slot_idx >= 0
        legacy = LegacyHandle(self._legacy_handle_tensors(ep_handle, is_token_in_rank, async_finish), ep_handle)
        return recv_x, recv_topk_idx, recv_topk_weights, ep_handle.num_recv_tokens_per_expert_list, legacy, event

    def _legacy_handle_tensors(self, ep_handle, is_token_in_rank, on_comm_stream: bool):
        """The six tensors of the reference's intranode handle (deep_ep/buffers/legacy.py:401), filled from what
        the dispatch left behind. There is one "channel" here (tokens are not cut into channel ranges):

        * ``rank_prefix_matrix[i, j]``: tokens that ranks ``0..i`` sent to rank ``j`` (the count exchange of the
          dispatch kernel gives every rank the whole matrix of totals);
        * ``channel_prefix_matrix[j, 0]``: tokens this rank sent to rank ``j``;
        * ``recv_channel_prefix_matrix[i, 0]``: tokens this rank received from rank ``i``;
        * ``recv_src_idx``, ``is_token_in_rank``;
        * ``send_head[t, j]``: position of token ``t`` among this rank's tokens for rank ``j`` (-1 = not sent).
        """
        R = self.group_size
        ctx = torch.cuda.stream(self.get_comm_stream()) if on_comm_stream else contextlib.nullcontext()
        with ctx:
            counts = ep_handle.num_tokens_per_rank_matrix      # [source, destination]
            rank_prefix_matrix = torch.cumsum(counts, dim=0).int()
            channel_prefix_matrix = counts[self.rank].clone().view(R, 1)
            recv_channel_prefix_matrix = counts[:, self.rank].clone().view(R, 1)
            slot = ep_handle.dst_buffer_slot_idx
            base = (rank_prefix_matrix[self.rank] - counts[self.rank]).view(1, R)
            send_head = torch.where(slot >= 0, slot - base, slot)
        return (rank_prefix_matrix, channel_prefix_matrix, recv_channel_prefix_matrix, ep_handle.recv_src_metadata[:, 0],
                is_token_in_rank, send_head)

    def combine(self, x: torch.Tensor, handle: Tuple, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[None, torch.Tensor, Tuple[torch.Tensor, torch.Tensor]] = None, config: Optional[Config] = None,
                previous_event: Optional[EventOverlap] = None, async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """Normal-mode combine: unweighted sum (+ bias). Returns ``(combined_x, combined_topk_weights, event)``."""
        config = config or self.get_combine_config(self.group_size)
        return self._elastic.combine(x, handle.ep_handle, topk_weights=topk_weights, bias=bias, num_sms=config.num_sms,
                                     previous_event=getattr(previous_event, 'event', None),
                                     async_with_compute_stream=async_finish, allocate_on_comm_stream=allocate_on_comm_stream)

    def internode_dispatch(self, *args, **kwargs):
        """One box, one tier: the same as :meth:`dispatch`."""
        return self.dispatch(*args, **kwargs)

    def internode_combine(self, *args, **kwargs):
        return self.combine(*args, **kwargs)

    # ------------------------------------------------------------------ low-latency mode
    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int, hidden: int, num_experts: int) -> None:
        """Flags are tagged with call counters and never need cleaning; this only orders the two modes
        (a barrier, so that no peer is still writing normal-mode rows into the shared heap)."""
        self._elastic.barrier()

    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int, num_experts: int,
                             cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                             dispatch_wait_recv_cost_stats: Optional[torch.Tensor] = None, use_fp8: bool = True,
                             round_scale: bool = False, use_ue8m0: bool = False, async_finish: bool = False,
                             return_recv_hook: bool = False, num_sms: int = 0):
        """Decode-batch dispatch into the expert-major packed layout.

        Returns ``(recv_x | (recv_x, recv_scales), recv_count, handle, event, hook)`` with
        ``recv_x [local experts, ranks * max tokens, hidden]``, scales column-major in their last two
        dimensions, ``recv_count [local experts]`` and
        ``handle = (src_info, layout_range, num_max_dispatch_tokens_per_rank, hidden, num_experts)``.
        With ``return_recv_hook`` only the sends are issued; ``hook()`` launches the receive part.
        """
        check_torch_deterministic()
        io = _C.LLDispatchIO()
        io.x, io.topk_idx = x, topk_idx
        io.cumulative_stats = cumulative_local_expert_recv_stats
        io.wait_stats = dispatch_wait_recv_cost_stats[self.rank] if dispatch_wait_recv_cost_stats is not None and \
            dispatch_wait_recv_cost_stats.dim() == 2 else dispatch_wait_recv_cost_stats
        phases = _C.LL_SEND if return_recv_hook else (_C.LL_SEND | _C.LL_RECV)
        args = (num_max_dispatch_tokens_per_rank, num_experts, use_fp8, round_scale, use_ue8m0)
        event = _C.ll_dispatch([self.runtime], [io], *args, phases, num_sms, self.enable_shrink, async_finish, return_recv_hook)
        hook: Optional[Callable] = None
        if return_recv_hook:
            def hook():
                _C.ll_dispatch([self.runtime], [io], *args, _C.LL_RECV, num_sms, self.enable_shrink, False, True)
        handle = (io.src_info, io.layout_range, num_max_dispatch_tokens_per_rank, x.size(1), num_experts)
        recv_x = (io.packed_recv_x, io.packed_recv_sf) if use_fp8 else io.packed_recv_x
        return recv_x, io.packed_recv_count, handle, EventOverlap(event), hook

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: tuple,
                            use_logfmt: bool = False, zero_copy: bool = False, async_finish: bool = False,
                            return_recv_hook: bool = False, out: Optional[torch.Tensor] = None,
                            combine_wait_recv_cost_stats: Optional[torch.Tensor] = None, num_sms: int = 0):
        """Weighted combine of the packed expert outputs: ``combined_x[t] = sum_k w[t, k] * x_k``.

        ``x`` is ``[local experts, ranks * max tokens, hidden]`` bf16 (with ``zero_copy`` it is the tensor
        from :meth:`get_next_low_latency_combine_buffer`). With ``use_logfmt`` every group of 128 channels whose
        largest magnitude is below 1 travels as 10-bit log-format values (160 instead of 256 bytes), the other
        groups stay bf16; ``deepep_b200.utils.math.logfmt_roundtrip`` restates the rounding. Returns
        ``(combined_x, event, hook)``. Reference: ``deep_ep/buffers/legacy.py:640-700``.
        """
        check_torch_deterministic()
        assert not (use_logfmt and zero_copy), 'LogFMT encodes while staging the row: it cannot be combined with zero_copy'
        src_info, layout_range, num_max_dispatch_tokens_per_rank, hidden, num_experts = handle
        io = _C.LLCombineIO()
        io.x, io.topk_idx, io.topk_weights = x, topk_idx, topk_weights
        io.src_info, io.layout_range = src_info, layout_range
        io.use_logfmt = bool(use_logfmt)
        if out is not None:
            io.combined_x = out
        io.wait_stats = combine_wait_recv_cost_stats[self.rank] if combine_wait_recv_cost_stats is not None and \
            combine_wait_recv_cost_stats.dim() == 2 else combine_wait_recv_cost_stats
        phases = _C.LL_SEND if return_recv_hook else (_C.LL_SEND | _C.LL_RECV)
        event = _C.ll_combine([self.runtime], [io], num_max_dispatch_tokens_per_rank, num_experts, phases, num_sms,
                              self.enable_shrink, async_finish, return_recv_hook)
        hook: Optional[Callable] = None
        if return_recv_hook:
            def hook():
                _C.ll_combine([self.runtime], [io], num_max_dispatch_tokens_per_rank, num_experts, _C.LL_RECV, num_sms,
                              self.enable_shrink, False, True)
        return io.combined_x, EventOverlap(event), hook

    def low_latency_update_mask_buffer(self, rank_to_mask: int, mask: bool = False):
        """Masks (or unmasks) a rank: nothing is sent to it and nothing is awaited from it."""
        _C.ll_mask_update(self.runtime, rank_to_mask, mask)

    def low_latency_query_mask_buffer(self, mask_status: torch.Tensor):
        """Fills ``mask_status [num_ranks]`` (int32) with 1 for masked ranks."""
        _C.ll_mask_query(self.runtime, mask_status)

    def low_latency_clean_mask_buffer(self):
        _C.ll_mask_clean(self.runtime)

    def get_next_low_latency_combine_buffer(self, handle: object):
        """bf16 ``[local experts, ranks * max tokens, hidden]`` staging tensor inside the heap that the next
        ``low_latency_combine(..., zero_copy=True)`` reads; let the expert GEMM write its output there."""
        _, _, num_max_dispatch_tokens_per_rank, hidden, num_experts = handle
        return _C.ll_next_combine_buffer(self.runtime, num_max_dispatch_tokens_per_rank, hidden, num_experts)
