"""Pipeline-parallel neighbour send / recv.

Two transports:

* :class:`PipelineRing` — slot rings in the symmetric heap (one ring per direction and rank).
  ``send`` waits (bounded) for the slot to be free, moves the tensor with a copy-engine
  ``cudaMemcpyAsync`` into the neighbour's ring and publishes a sequence number; ``recv`` waits for
  it, copies the slot out and acknowledges. A send never needs a matching receive to be posted, so
  any interleaving of sends and receives with at most ``num_max_inflight_tensors`` outstanding is
  deadlock free. All work runs on the communication stream and overlaps with compute.
* :func:`nccl_send_recv` — the same exchange as one batched NCCL point-to-point group on a side
  stream, for pipelines that pair their sends and receives.

Parity: csrc/elastic/buffer.hpp:327-375 and deep_ep/include/deep_ep/impls/pp_send_recv.cuh of the
reference (pp_set_config / pp_send / pp_recv over a slot ring with signals).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .._native import _C


def _align(x: int, a: int = 256) -> int:
    return -(-x // a) * a


class PipelineRing:
    def __init__(self, buffer):
        self.buffer, self.rt = buffer, buffer.runtime
        self.rank, self.num_ranks = buffer.rank_idx, buffer.num_ranks
        self.prev, self.next = (self.rank - 1) % self.num_ranks, (self.rank + 1) % self.num_ranks
        self.num_max_tensor_bytes = 0
        self.num_slots = 0
        self.send_seq = [0, 0]
        self.recv_seq = [0, 0]

    def set_config(self, num_max_tensor_bytes: int, num_max_inflight_tensors: int) -> None:
        assert 1 <= num_max_inflight_tensors <= 64
        need = int(_C.CONTROL_BYTES) + 2 * num_max_inflight_tensors * _align(num_max_tensor_bytes)
        assert need <= self.rt.num_bytes(), 'buffer too small for this PP configuration'
        self.num_max_tensor_bytes, self.num_slots = num_max_tensor_bytes, num_max_inflight_tensors

    def _slot_off(self, direction: int, slot: int) -> int:
        return int(_C.CONTROL_BYTES) + (direction * self.num_slots + slot) * _align(self.num_max_tensor_bytes)

    @staticmethod
    def _word(direction: int, kind: int, slot: int) -> int:
        return int(_C.CTL_PP_SIGNALS) + ((direction * 2 + kind) * 64 + slot) * 8

    # direction as the RECEIVER sees it: 0 = from its previous rank, 1 = from its next rank
    def send(self, t: torch.Tensor, dst_rank_idx: int) -> None:
        PipelineRing.multi_send([self], [t], [dst_rank_idx])

    def recv(self, t: torch.Tensor, src_rank_idx: int) -> None:
        PipelineRing.multi_recv([self], [t], [src_rank_idx])

    @staticmethod
    def multi_send(rings: List['PipelineRing'], tensors: Sequence[torch.Tensor], dsts: Sequence[int]) -> None:
        comm = rings[0].buffer.get_comm_stream()
        comm.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(comm):
            waits, signals, plan = [], [], []
            for r, t, dst in zip(rings, tensors, dsts):
                assert r.num_slots > 0, 'call pp_set_config first'
                assert t.is_cuda and t.is_contiguous() and t.numel() * t.element_size() <= r.num_max_tensor_bytes
                assert dst in (r.next, r.prev), 'PP sends go to the previous or the next rank'
                direction = 0 if dst == r.next else 1
                r.send_seq[direction] += 1
                seq = r.send_seq[direction]
                slot = (seq - 1) % r.num_slots
                w = _C.FlagSpec()
                if seq > r.num_slots:     # the receiver must have consumed the tensor that used this slot before
                    w.wait_offsets = [PipelineRing._word(direction, 1, slot)]
                    w.wait_value = seq - r.num_slots
                w.status_code = int(_C.STATUS_PP)
                s = _C.FlagSpec()
                s.signals = [(dst, PipelineRing._word(direction, 0, slot))]
                s.signal_value = seq
                s.status_code = int(_C.STATUS_PP)
                waits.append(w)
                signals.append(s)
                plan.append((r, t, dst, r._slot_off(direction, slot)))
            rts = [r.rt for r in rings]
            _C.flag_op(rts, waits)
            for r, t, dst, off in plan:
                _C.copy_to_heap(r.rt, dst, off, t)
            _C.flag_op(rts, signals)
        for t in tensors:
            t.record_stream(comm)

    @staticmethod
    def multi_recv(rings: List['PipelineRing'], tensors: Sequence[torch.Tensor], srcs: Sequence[int]) -> None:
        comm = rings[0].buffer.get_comm_stream()
        compute = torch.cuda.current_stream()
        comm.wait_stream(compute)
        with torch.cuda.stream(comm):
            waits, signals, plan = [], [], []
            for r, t, src in zip(rings, tensors, srcs):
                assert r.num_slots > 0, 'call pp_set_config first'
                assert t.is_cuda and t.is_contiguous() and t.numel() * t.element_size() <= r.num_max_tensor_bytes
                assert src in (r.prev, r.next), 'PP receives come from the previous or the next rank'
                direction = 0 if src == r.prev else 1
                r.recv_seq[direction] += 1
                seq = r.recv_seq[direction]
                slot = (seq - 1) % r.num_slots
                w = _C.FlagSpec()
                w.wait_offsets = [PipelineRing._word(direction, 0, slot)]
                w.wait_value = seq
                w.status_code = int(_C.STATUS_PP)
                s = _C.FlagSpec()
                s.signals = [(src, PipelineRing._word(direction, 1, slot))]
                s.signal_value = seq
                s.status_code = int(_C.STATUS_PP)
                waits.append(w)
                signals.append(s)
                plan.append((r, t, r._slot_off(direction, slot)))
            rts = [r.rt for r in rings]
            _C.flag_op(rts, waits)
            for r, t, off in plan:
                _C.copy_from_heap(r.rt, off, t)
            _C.flag_op(rts, signals)
        compute.wait_stream(comm)


def nccl_send_recv(send: Optional[torch.Tensor], dst: Optional[int], recv: Optional[torch.Tensor], src: Optional[int],
                   group: Optional[dist.ProcessGroup] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.cuda.Event:
    """One batched NCCL p2p group (send and/or recv) on ``stream``; returns the event that marks its end."""
    stream = stream or torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    ops = []
    if send is not None:
        ops.append(dist.P2POp(dist.isend, send, dst, group=group))
    if recv is not None:
        ops.append(dist.P2POp(dist.irecv, recv, src, group=group))
    with torch.cuda.stream(stream):
        for work in dist.batch_isend_irecv(ops):
            work.wait()
        done = torch.cuda.Event()
        done.record(stream)
    for t in (send, recv):
        if t is not None:
            t.record_stream(stream)
    return done
