"""Stream-overlap sugar around the native event handle.

Parity: deep_ep/utils/event.py:8-96 of the reference (``EventOverlap``: ``current_stream_wait``,
``with`` blocks, and a hook that runs after the wait).
"""
from __future__ import annotations

from typing import Any, Callable, Optional, Tuple

import torch


class EventOverlap:
    """Wraps the event returned by an asynchronous communication call.

    Usage::

        recv_x, ..., event = buffer.dispatch(..., async_with_compute_stream=True)
        with event:           # the current stream waits for the event when the block ends
            do_unrelated_compute()

    Attributes:
        event: the native event handle (``None`` for synchronous calls).
        extra_tensors: tensors kept alive until the event is waited for.
    """

    def __init__(self, event: Optional[Any] = None, extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None) -> None:
        self.event = event
        self.extra_tensors = extra_tensors
        self._hook: Optional[Callable[[], None]] = None

    def current_stream_wait(self, release_handle: bool = False) -> None:
        """Makes the current stream wait for the communication to finish, then runs the hook once."""
        if self.event is not None:
            self.event.current_stream_wait()
        if self._hook is not None:
            hook, self._hook = self._hook, None
            hook()
        if release_handle:
            self.event = None
            self.extra_tensors = None

    def register_hook_after_wait(self, hook: Callable[[], None]) -> None:
        """``hook`` runs right after the first wait (the deterministic sort of a handle uses this)."""
        assert self._hook is None, 'only one hook is supported'
        self._hook = hook

    def __call__(self, release_handle: bool = False) -> 'EventOverlap':
        self._release_on_exit = release_handle
        return self

    def __enter__(self) -> 'EventOverlap':
        return self

    def __exit__(self, exc_type, exc_val, exc_tb) -> None:
        self.current_stream_wait(release_handle=getattr(self, '_release_on_exit', False))
