"""Loads the in-tree native extension ``deepep_b200._C``.

The shared object is built by ``python -m deepep_b200._build`` and lives next to this file.
On a machine with a GPU a missing extension is an error at import time (there is no eager
fallback for the communication kernels); without a GPU the pure-Python parts of the package
(oracle, gate generators, SM model helpers) stay importable.
"""
from __future__ import annotations

import torch

try:
    from . import _C  # type: ignore[attr-defined]
    _IMPORT_ERROR = None
except ImportError as exc:  # pragma: no cover - depends on the build state
    _C = None
    _IMPORT_ERROR = exc
    if torch.cuda.is_available():
        raise RuntimeError('deepep_b200._C is missing or does not load on a machine with a GPU; '
                           'build it with `python -m deepep_b200._build`') from exc


def require_native():
    """Returns the native module or raises with the build instruction."""
    if _C is None:
        raise RuntimeError(f'deepep_b200._C is not built ({_IMPORT_ERROR}); run `python -m deepep_b200._build`')
    return _C
