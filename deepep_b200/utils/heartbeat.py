"""Host-side failure detection: a store-based heartbeat between the ranks of a job.

Device waits in this library are bounded and report a status instead of hanging, but a rank that
has died is better noticed BEFORE the next collective launch. Every rank publishes a monotonically
increasing beat under ``hb/<rank>`` in a ``torch.distributed`` store (TCPStore / FileStore);
:meth:`Heartbeat.dead_ranks` lists the peers whose beat has not advanced for ``timeout`` seconds.
A caller in shrink mode then masks those ranks (``Buffer.low_latency_update_mask_buffer``); others
raise and rebuild their buffers.

Parity: the reference detects failures only on the device (timeouts that trap, or the low-latency
mask buffer, csrc/kernels/legacy/internode_ll.cu:10-69); this is the host-side complement.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, interval: float = 0.2, timeout: float = 2.0, autostart: bool = True):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.interval, self.timeout = interval, timeout
        self._beat = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, tuple] = {}
        self.beat()
        if autostart:
            self.start()

    def beat(self) -> None:
        self._beat += 1
        self.store.set(f'hb/{self.rank}', str(self._beat))

    def start(self) -> None:
        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:   # the store is gone: the job is ending
                    return
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def dead_ranks(self) -> List[int]:
        """Peers whose beat has not advanced within ``timeout`` seconds (since this method first saw it)."""
        now = time.time()
        dead = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            try:
                value = int(self.store.get(f'hb/{r}'))
            except Exception:
                value = -1
            last = self._seen.get(r)
            if last is None or last[0] != value:
                self._seen[r] = (value, now)
            elif now - last[1] > self.timeout:
                dead.append(r)
        return dead
