"""All-gather / reduce-scatter sessions on the symmetric heap ("AGRS", also the context-parallel
chunk all-gather).

Payload moves on the copy engines: every rank issues one ``cudaMemcpyAsync`` per peer into that
peer's heap, each on a side stream forked from the communication stream so that the copies to
different peers run on different copy engines; no SM is used for the transfer. Arrival is published
and awaited by a one-block flag kernel (bounded wait). Gathered tensors are views of the heap with a
leading ``num_ranks`` dimension; a session bounds the life of those views, and ending a session
tells the peers that this rank is done reading, which is what allows the next session to overwrite
the area.

Parity: csrc/elastic/buffer.hpp:377-524 of the reference (agrs_set_config, sessions,
agrs_get_inplace_tensor, all_gather). ``reduce_scatter`` has no counterpart there (listed as
not implemented in the reference's README).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple, Union

import torch

from .._native import _C


def _align(x: int, a: int = 256) -> int:
    return -(-x // a) * a


class AgrsManager:
    """Session bookkeeping of one rank. ``multi_*`` static methods take the managers of all virtual
    ranks of a single-GPU emulation and issue their flag kernels as one cooperative launch."""

    RELEASE_ROW = None  # set from the native constant on first use

    def __init__(self, buffer):
        self.buffer = buffer
        self.rt = buffer.runtime
        self.rank, self.num_ranks = buffer.rank_idx, buffer.num_ranks
        self.base = int(_C.CONTROL_BYTES)
        self.num_max_session_bytes = (self.rt.num_bytes() - self.base) // self.num_ranks // 256 * 256
        self.num_max_all_gathers = int(_C.MAX_AGRS_INFLIGHT)
        self.session_idx = 0
        self.active = False
        self.offset = 0
        self.ag_idx = 0
        self.waited_release = True
        self.pending_inplace = {}

    # ------------------------------------------------------------------ configuration / sessions
    def set_config(self, num_max_session_bytes: int, num_max_all_gathers_per_session: int) -> None:
        assert not self.active
        assert num_max_all_gathers_per_session <= int(_C.MAX_AGRS_INFLIGHT)
        assert self.base + self.num_ranks * _align(num_max_session_bytes) <= self.rt.num_bytes(), 'buffer too small for this session size'
        self.num_max_session_bytes = num_max_session_bytes
        self.num_max_all_gathers = num_max_all_gathers_per_session

    def create_session(self) -> None:
        assert not self.active, 'the previous AGRS session is still open'
        self.session_idx += 1
        self.active, self.offset, self.ag_idx = True, 0, 0
        self.waited_release = self.session_idx == 1
        self.pending_inplace = {}

    def _signal_off(self, row: int, rank: int) -> int:
        return int(_C.CTL_AGRS_SIGNALS) + (row * int(_C.MAX_RANKS) + rank) * 8

    def _reserve(self, nbytes: int) -> int:
        assert self.active, 'open an AGRS session first'
        assert self.ag_idx + 0 <= self.num_max_all_gathers
        off = self.offset
        self.offset += self.num_ranks * _align(nbytes)
        assert self.offset <= self.num_ranks * _align(self.num_max_session_bytes), 'AGRS session buffer exhausted'
        return self.base + off

    def get_inplace_tensor(self, shapes, dtype: torch.dtype):
        """Tensor(s) that live in this rank's slot of the coming all-gather(s): fill them, then pass them to
        :meth:`all_gather`, which then has nothing to copy locally."""
        batched = isinstance(shapes[0], (tuple, list, torch.Size))
        shape_list = list(shapes) if batched else [shapes]
        out = []
        for shape in shape_list:
            nbytes = math.prod(shape) * torch.empty(0, dtype=dtype).element_size()
            region = self._reserve(nbytes)
            t = self.rt.heap_tensor(region + self.rank * _align(nbytes), nbytes).view(dtype).view(*shape)
            self.pending_inplace[t.data_ptr()] = (region, nbytes)
            out.append(t)
        return tuple(out) if batched else out[0]

    def destroy_session(self) -> None:
        AgrsManager.multi_destroy([self])

    # ------------------------------------------------------------------ collectives
    def all_gather(self, t: Union[torch.Tensor, Sequence[torch.Tensor]]):
        return AgrsManager.multi_all_gather([self], [t])[0]

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        return AgrsManager.multi_reduce_scatter([self], [t])[0]

    # ------------------------------------------------------------------ multi-rank forms
    @staticmethod
    def _streams(mgrs):
        comm = mgrs[0].buffer.get_comm_stream()
        compute = torch.cuda.current_stream()
        return comm, compute

    @staticmethod
    def _flag_round(mgrs: List['AgrsManager'], row: int, wait: bool = True, signal: bool = True, value: Optional[int] = None) -> None:
        specs = []
        for m in mgrs:
            s = _C.FlagSpec()
            v = m.session_idx if value is None else value
            if signal:
                s.signals = [(p, m._signal_off(row, m.rank)) for p in range(m.num_ranks)]
                s.signal_value = v
            if wait:
                s.wait_offsets = [m._signal_off(row, p) for p in range(m.num_ranks)]
                s.wait_value = v
            s.status_code = int(_C.STATUS_AGRS)
            s.signal_first = True     # an arrival round: publish the own arrival, then wait for the peers'
            specs.append(s)
        _C.flag_op([m.rt for m in mgrs], specs)

    @staticmethod
    def _wait_release(mgrs: List['AgrsManager']) -> None:
        """Before the first write of a session: every peer must have ended the previous session."""
        if all(m.waited_release for m in mgrs):
            return
        AgrsManager._flag_round(mgrs, int(_C.MAX_AGRS_INFLIGHT), wait=True, signal=False, value=mgrs[0].session_idx - 1)
        for m in mgrs:
            m.waited_release = True

    @staticmethod
    def multi_all_gather(mgrs: List['AgrsManager'], tensors_per_rank):
        comm, compute = AgrsManager._streams(mgrs)
        comm.wait_stream(compute)
        results = []
        with torch.cuda.stream(comm):
            AgrsManager._wait_release(mgrs)
            for m, ts in zip(mgrs, tensors_per_rank):
                single = isinstance(ts, torch.Tensor)
                ts = [ts] if single else list(ts)
                gathered = []
                for t in ts:
                    assert t.is_cuda and t.is_contiguous()
                    nbytes = t.numel() * t.element_size()
                    inplace = m.pending_inplace.pop(t.data_ptr(), None)
                    region = inplace[0] if inplace is not None else m._reserve(nbytes)
                    slot = _align(nbytes)
                    # peers first, starting behind this rank (no two ranks begin with the same target), own slot last
                    order = [(m.rank + 1 + i) % m.num_ranks for i in range(m.num_ranks)]
                    _C.copy_fanout(m.rt, [(p, region + m.rank * slot, t) for p in order if not (p == m.rank and inplace is not None)])
                    if slot == nbytes:
                        view = m.rt.heap_tensor(region, m.num_ranks * slot).view(t.dtype).view(m.num_ranks, *t.shape)
                    else:   # padded slots: a strided view
                        view = m.rt.heap_tensor(region, m.num_ranks * slot).view(m.num_ranks, slot)[:, :nbytes].view(t.dtype) \
                            .view(m.num_ranks, *t.shape)
                    gathered.append(view)
                results.append((single, gathered))
            row = mgrs[0].ag_idx
            assert row < int(_C.MAX_AGRS_INFLIGHT)
            AgrsManager._flag_round(mgrs, row)
            for m in mgrs:
                m.ag_idx += 1
            done = torch.cuda.Event()
            done.record(comm)

        def handle() -> None:
            torch.cuda.current_stream().wait_event(done)

        out = []
        for single, gathered in results:
            out.append((gathered[0], handle) if single else (*gathered, handle))
        return out

    @staticmethod
    def multi_reduce_scatter(mgrs: List['AgrsManager'], tensors: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        """``out_r = sum_s tensors[s][chunk r]`` (fp32 accumulation in rank order); leading dim divisible by ranks."""
        comm, compute = AgrsManager._streams(mgrs)
        comm.wait_stream(compute)
        outs = []
        implicit = [not m.active for m in mgrs]
        for m, imp in zip(mgrs, implicit):
            if imp:
                m.create_session()
        with torch.cuda.stream(comm):
            AgrsManager._wait_release(mgrs)
            regions = []
            for m, t in zip(mgrs, tensors):
                assert t.is_cuda and t.is_contiguous() and t.size(0) % m.num_ranks == 0 and t.dtype in (torch.bfloat16, torch.float32)
                chunks = t.view(m.num_ranks, -1)
                nbytes = chunks[0].numel() * t.element_size()
                assert nbytes % 16 == 0
                region = m._reserve(nbytes)
                order = [(m.rank + 1 + i) % m.num_ranks for i in range(m.num_ranks)]
                _C.copy_fanout(m.rt, [(p, region + m.rank * _align(nbytes), chunks[p]) for p in order])
                regions.append((region, nbytes))
            AgrsManager._flag_round(mgrs, mgrs[0].ag_idx)
            for m, t, (region, nbytes) in zip(mgrs, tensors, regions):
                m.ag_idx += 1
                out = torch.empty((t.size(0) // m.num_ranks, *t.shape[1:]), dtype=t.dtype, device=t.device)
                _C.reduce_slots(m.rt, region, _align(nbytes), m.num_ranks, out)
                outs.append(out)
        compute.wait_stream(comm)
        for m, imp in zip(mgrs, implicit):
            if imp:
                pass
        if any(implicit):
            AgrsManager.multi_destroy([m for m, imp in zip(mgrs, implicit) if imp])
        return outs

    @staticmethod
    def multi_destroy(mgrs: List['AgrsManager']) -> None:
        comm, compute = AgrsManager._streams(mgrs)
        comm.wait_stream(compute)      # the compute stream has finished reading the gathered views
        with torch.cuda.stream(comm):
            AgrsManager._flag_round(mgrs, int(_C.MAX_AGRS_INFLIGHT), wait=False, signal=True)
        for m in mgrs:
            m.active = False
            m.pending_inplace = {}
