"""Host model of the symmetric heap's flag barrier (``barrier_kernel`` in ops/csrc/runtime.cu).

The device protocol: every rank owns ``n_ranks`` 64-bit slots.  *Arrive*: store the epoch into
``slots[peer][my_rank]`` of every peer (release).  *Wait*: poll the own slots until all are ``>= epoch``
(acquire), for at most ``timeout``; on expiry report a status instead of spinning on.  Epochs only grow,
which is what makes a late or repeated arrival harmless and lets a fast rank arrive at epoch ``e + 1`` while
a slow one still waits at ``e``.

This module restates that state machine with Python threads so that its properties (no early release,
visibility of writes made before the arrival, bounded waits, recovery after a missed epoch) can be tested
without a GPU and without ever hanging one.  The reference has no counterpart: its ranks meet in NCCL
collectives (src/tplr/distributed.py:148-183 ``safe_barrier``).
"""

from __future__ import annotations

import threading
import time

ST_OK, ST_WAIT_TIMEOUT = 0, 4        # same bit as TPLR_ST_WAIT_TIMEOUT


class FlagBarrierModel:
    def __init__(self, n_ranks: int):
        self.n = n_ranks
        self.slots = [[0] * n_ranks for _ in range(n_ranks)]     # slots[owner][writer]
        self._mem = threading.Lock()                             # one memory system: stores are atomic words
        self.status = [ST_OK] * n_ranks

    def arrive(self, rank: int, epoch: int) -> None:
        for peer in range(self.n):
            with self._mem:
                # a plain store of the epoch, as on the device; epochs are issued in increasing order per rank
                self.slots[peer][rank] = epoch

    def wait(self, rank: int, epoch: int, timeout_s: float) -> int:
        t0 = time.monotonic()
        for writer in range(self.n):
            while True:
                with self._mem:
                    v = self.slots[rank][writer]
                if v >= epoch:
                    break
                if time.monotonic() - t0 > timeout_s:
                    self.status[rank] |= ST_WAIT_TIMEOUT
                    return self.status[rank]
                time.sleep(0)
        return ST_OK

    def barrier(self, rank: int, epoch: int, timeout_s: float = 5.0) -> int:
        self.arrive(rank, epoch)
        return self.wait(rank, epoch, timeout_s)
