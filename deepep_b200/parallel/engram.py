"""Engram: a table of rows sharded over the ranks' heaps, fetched by index from any rank.

``write`` places this rank's shard in its heap; ``fetch`` launches a kernel on the communication
stream that pulls every requested row from its owner's memory with a plain bulk load over NVLink
(no multicast) and stores it locally, and returns a hook that makes the caller's stream wait and
hands out the rows. FP8 tables carry a replicated per-entry scale table that is gathered locally.

With ``num_cpu_bytes > 0`` on the buffer the shards live in the ranks' pinned host segments instead
(``ElasticBuffer.host_segments``), as in the reference: ``write`` copies the shard to the rank's own
segment, ``fetch`` reads the owners' segments with plain loads over PCIe.

Parity: csrc/elastic/buffer.hpp:210-325 and impls/engram_fetch*.cuh of the reference (which issues
RDMA gets for remote nodes and loads for the machine's own host segments).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch

from .._native import _C


class EngramStore:
    def __init__(self, buffer):
        self.buffer, self.rt = buffer, buffer.runtime
        self.rank, self.num_ranks = buffer.rank_idx, buffer.num_ranks
        self.table_offset = int(_C.CONTROL_BYTES)
        self.entries_per_rank = 0
        self.hidden = 0
        self.dtype = torch.bfloat16
        self.sf: Optional[torch.Tensor] = None

    @property
    def on_host(self) -> bool:
        return len(getattr(self.buffer, 'host_segments', [])) == self.num_ranks and self.buffer.num_cpu_bytes > 0

    def write(self, storage: torch.Tensor, sf: Optional[torch.Tensor] = None, barrier: bool = True) -> None:
        assert storage.is_cuda and storage.dim() == 2 and storage.is_contiguous()
        assert storage.dtype in (torch.bfloat16, torch.float8_e4m3fn)
        assert (sf is not None) == (storage.dtype == torch.float8_e4m3fn), 'scales go with FP8 storage and only with it'
        self.entries_per_rank, self.hidden, self.dtype = storage.size(0), storage.size(1), storage.dtype
        if barrier:
            self.buffer.barrier()
        if self.on_host:
            assert storage.numel() * storage.element_size() <= self.buffer.num_cpu_bytes, 'Engram storage exceeds the CPU segment'
            self.buffer.host_segments[self.rank].copy_from_device(storage.view(torch.uint8), 0)
            torch.cuda.current_stream().synchronize()      # the barrier below is a device-side handshake only
        else:
            _C.copy_to_heap(self.rt, self.rank, self.table_offset, storage.view(torch.uint8))
        self.sf = sf.contiguous() if sf is not None else None
        if barrier:
            self.buffer.barrier()

    def fetch(self, indices: torch.Tensor, use_tma_aligned_col_major_sf: bool = False, num_sms: int = 0) -> Callable:
        return EngramStore.multi_fetch([self], [indices], use_tma_aligned_col_major_sf, num_sms)[0]

    @staticmethod
    def multi_fetch(stores: List['EngramStore'], indices: Sequence[torch.Tensor], col_major_sf: bool = False,
                    num_sms: int = 0) -> List[Callable]:
        s0 = stores[0]
        comm = s0.buffer.get_comm_stream()
        comm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(comm):
            res = _C.engram_gather([s.rt for s in stores], [i.contiguous() for i in indices], s0.table_offset, s0.entries_per_rank,
                                   s0.hidden, s0.dtype, [s.sf for s in stores], col_major_sf, num_sms,
                                   [list(s.buffer.host_segments) for s in stores] if s0.on_host else [])
            done = torch.cuda.Event()
            done.record(comm)
        hooks = []
        for data, sf in res:
            def hook(data=data, sf=sf):
                torch.cuda.current_stream().wait_event(done)
                return data, sf
            hooks.append(hook)
        return hooks
