"""Process-group helpers: a cache of per-group communication resources.

The reference keeps a cache of NCCL communicator handles per process group because its device code
talks to NCCL's symmetric windows (deep_ep/utils/comm.py:11-83). Here the data plane is an own
symmetric heap, so what is cached per group is the ``ElasticBuffer`` itself; NCCL is only used
through ``torch.distributed`` for bootstrap and baselines.
"""
from __future__ import annotations

import weakref
from typing import Any, Dict, Tuple

_buffers: Dict[Tuple[int, Tuple], Any] = {}


def get_cached_buffer(group: Any, **buffer_kwargs):
    """One ``ElasticBuffer`` per (group, settings): repeated layers of a model share the heap."""
    from ..buffers.elastic import ElasticBuffer
    key = (id(group), tuple(sorted(buffer_kwargs.items())))
    buf = _buffers.get(key)
    if buf is None or getattr(buf, '_destroyed', True):
        buf = ElasticBuffer(group, **buffer_kwargs)
        _buffers[key] = buf
    return buf


def destroy_all_cached_buffers() -> None:
    for buf in list(_buffers.values()):
        try:
            buf.destroy()
        except Exception:   # already gone
            pass
    _buffers.clear()
