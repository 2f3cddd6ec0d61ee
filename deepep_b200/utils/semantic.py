"""Small semantic helpers.

Parity: deep_ep/utils/semantic.py:5-27 of the reference (``value_or``, ``weak_lru``).
"""
from __future__ import annotations

import functools
import weakref
from typing import Any, Callable, Optional


def value_or(value: Optional[Any], default: Any) -> Any:
    """``value`` unless it is ``None``."""
    return value if value is not None else default


def weak_lru(maxsize: Optional[int] = 128, typed: bool = False) -> Callable:
    """``functools.lru_cache`` for methods that does not keep ``self`` alive.

    The cache key holds a weak reference to the instance, so a cached method never
    extends the life of a buffer object (and of the device memory behind it).
    """

    def decorate(method: Callable) -> Callable:
        @functools.lru_cache(maxsize=maxsize, typed=typed)
        def cached(ref, *args, **kwargs):
            return method(ref(), *args, **kwargs)

        @functools.wraps(method)
        def bound(self, *args, **kwargs):
            return cached(weakref.ref(self), *args, **kwargs)

        bound.cache_clear = cached.cache_clear  # type: ignore[attr-defined]
        return bound

    return decorate
