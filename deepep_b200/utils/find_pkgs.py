"""Locates the roots of the CUDA toolkit and of optional NVIDIA packages (NCCL headers for
baselines). Order: ``EP_<NAME>_ROOT_DIR`` / ``<NAME>_DIR`` / ``<NAME>_HOME`` environment variables,
then pip ``nvidia-*`` wheels in ``sys.path`` order, then well-known system paths.

Parity: deep_ep/utils/find_pkgs.py:8-82 of the reference. NVSHMEM is not used by this library;
asking for it returns ``None``.
"""
from __future__ import annotations

import os
import sys
from typing import Optional


def find_pkg_root(name: str, lib_name: Optional[str] = None, optional: bool = False) -> Optional[str]:
    upper = name.upper()
    for key in (f'EP_{upper}_ROOT_DIR', f'{upper}_DIR', f'{upper}_HOME', f'{upper}_ROOT'):
        path = os.environ.get(key)
        if path and os.path.isdir(path):
            return path
    for base in sys.path:
        cand = os.path.join(base, 'nvidia', name.lower())
        if os.path.isdir(cand) and (lib_name is None or os.path.isdir(os.path.join(cand, 'lib'))):
            return cand
    for cand in (f'/usr/local/{name.lower()}', f'/opt/{name.lower()}'):
        if os.path.isdir(cand):
            return cand
    if optional:
        return None
    raise FileNotFoundError(f'cannot find {name}; set EP_{upper}_ROOT_DIR')


def find_cuda_home() -> str:
    for key in ('CUDA_HOME', 'CUDA_PATH'):
        if os.environ.get(key):
            return os.environ[key]
    return find_pkg_root('cuda', optional=True) or '/usr/local/cuda'


def find_nccl_root(optional: bool = True) -> Optional[str]:
    return find_pkg_root('nccl', 'libnccl.so.2', optional=optional)


def find_nvshmem_root(optional: bool = True) -> Optional[str]:
    """NVSHMEM is not a dependency of this library."""
    return None
