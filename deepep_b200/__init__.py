"""B200-native expert-parallel communication library.

Public surface (names follow deep_ep/__init__.py:88-97 of the reference):
``ElasticBuffer``, ``EPHandle``, ``Buffer``, ``Config``, ``EventOverlap``, ``EventHandle``,
``topk_idx_t``, ``get_physical_domain_size``, ``get_logical_domain_size``.
"""
from __future__ import annotations

import os

# defaults fixed when the package was built (setup.py writes deepep_b200/envs.py); the process environment wins
try:
    from .envs import persistent_envs as _persistent_envs
    for _key, _value in _persistent_envs.items():
        os.environ.setdefault(_key, _value)
except ImportError:
    pass

import torch

from ._native import _C, require_native  # noqa: F401
from .buffers.elastic import ElasticBuffer, EPHandle  # noqa: F401
from .buffers.legacy import Buffer, Config  # noqa: F401
from .utils.envs import get_logical_domain_size, get_physical_domain_size  # noqa: F401
from .utils.event import EventOverlap  # noqa: F401

# dtype of routing indices the caller is expected to pass (the kernels accept both at run time); the reference
# fixes it at build time with EP_NUM_TOPK_IDX_BITS (deep_ep/include/deep_ep/common/compiled.cuh:54-72)
topk_idx_t = torch.int32 if os.environ.get('EP_NUM_TOPK_IDX_BITS', '64') == '32' else torch.int64
EventHandle = _C.EventHandle if _C is not None else None
EPException = _C.EPException if _C is not None else RuntimeError
EPTimeoutError = _C.EPTimeoutError if _C is not None else TimeoutError

__version__ = '0.1.0'
