"""Run-time specialisation of kernels (hidden size, top-k, rank count as compile-time constants).

``build(name, code)`` compiles a ``.cu`` source string whose single kernel is called
``ep_jit_entry`` and takes one parameter block by value; the cubin is cached on disk under
``$EP_JIT_CACHE_DIR`` (default ``~/.deepep_b200/cache``) keyed by the code, the flags, the compiler
version and the content of the included library headers. ``launch`` loads it (once per process) and
starts it on the current stream. The native part lives in ``csrc/jit/jit.hpp``.

Environment: ``EP_JIT_CACHE_DIR``, ``EP_JIT_NVCC_COMPILER``, ``EP_JIT_CPP_STANDARD``,
``EP_JIT_PRINT_COMPILER_COMMAND``, ``EP_JIT_DEBUG``, ``EP_JIT_PTXAS_VERBOSE``, ``EP_JIT_PTXAS_CHECK``,
``EP_JIT_WITH_LINEINFO``. The reference's assembly dump options (``EP_JIT_DUMP_ASM/PTX/SASS``) are not
offered.

Parity: csrc/jit/ of the reference and ``init_jit`` in deep_ep/__init__.py:71-84.
"""
from __future__ import annotations

import os
import struct
from pathlib import Path
from typing import Sequence, Tuple

from .._native import require_native
from ..utils.find_pkgs import find_cuda_home

_initialised = False
INCLUDE_ROOT = str(Path(__file__).resolve().parent.parent / 'csrc')


def init(cache_dir: str = '', include_root: str = '') -> None:
    """Sets the cache directory and the root of the library headers that JIT sources may include (default: the
    ``csrc`` tree of the installed package). The content of every included header is part of the cache key."""
    global _initialised
    C = require_native()
    cache_dir = cache_dir or os.environ.get('EP_JIT_CACHE_DIR') or os.path.join(os.path.expanduser('~'), '.deepep_b200', 'cache')
    C.jit_init(cache_dir, find_cuda_home(), include_root or INCLUDE_ROOT)
    _initialised = True


def build(name: str, code: str) -> str:
    """Compiles (or finds in the cache) and returns the cubin path."""
    if not _initialised:
        init()
    return require_native().jit_build(name, code)


def launch(cubin: str, grid: Sequence[int], block: Sequence[int], params: bytes, smem_bytes: int = 0, cooperative: bool = False,
           cluster_dim: int = 1) -> None:
    g = tuple(list(grid) + [1] * (3 - len(grid)))
    b = tuple(list(block) + [1] * (3 - len(block)))
    require_native().jit_launch(cubin, g, b, smem_bytes, params, cooperative, cluster_dim)


def pack(fmt: str, *values) -> bytes:
    """``struct.pack`` with native alignment: the by-value parameter block of a JIT kernel."""
    return struct.pack('@' + fmt, *values)


def combine_reduce_source(hidden: int, num_lanes: int) -> str:
    """Source of the combine reduction specialised for a hidden size and a lane count (fully unrolled
    row loop, 16-byte loads of all lanes in flight before the first add)."""
    return f'''
#include "kernels/jit/combine_reduce_jit.cuh"
extern "C" __global__ void __launch_bounds__(256) ep_jit_entry(const __grid_constant__ ep::jit::CombineReduceParams p) {{
    ep::jit::combine_reduce<{hidden}, {num_lanes}>(p);
}}
'''
