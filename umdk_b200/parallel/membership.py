"""Who is still there: a host-side membership view for the ranks of a job, kept in a key-value store.

The device kernels of this package wait on flags that peers write, with a bounded budget (they return a status
instead of hanging). That bounds the damage of a missing peer; this module avoids it: a rank that leaves says so
BETWEEN steps, a rank that dies stops refreshing its heartbeat, and every rank looks at the view before it launches
the next step, so no kernel is ever launched against a rank that is known to be gone. The reference has no
counterpart for its device operators (their waits are unbounded spins, e.g. moe_dispatch_normal.h:495); its host
libraries do the same job with keepalive probes (src/urpc/framework/lib/manager/keepalive.h) and TCP keepalive in
the lock server (src/ulock/dlock/lib/server/dlock_server.cpp).
"""
from __future__ import annotations

import time
from typing import Iterable, List, Optional, Set


class Membership:
    """View over `world` ranks in a `torch.distributed` store (TCPStore / FileStore / HashStore).

    `beat()` refreshes this rank's heartbeat, `leave()` announces an orderly departure, `alive()` returns the ranks
    that have neither left nor been silent for longer than `timeout_s`."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "umdk/member"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self._left = False
        self.beat()

    def _key(self, kind: str, r: int) -> str:
        return f"{self.prefix}/{kind}/{r}"

    def beat(self) -> None:
        if not self._left:
            self.store.set(self._key("beat", self.rank), repr(time.time()))

    def leave(self) -> None:
        """Orderly departure: call between steps, with no kernel or collective of this rank in flight."""
        self._left = True
        self.store.set(self._key("left", self.rank), "1")

    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:  # a store that cannot answer tells us nothing about the rank
            return None

    def alive(self, ranks: Optional[Iterable[int]] = None) -> Set[int]:
        now = time.time()
        out = set()
        for r in (range(self.world) if ranks is None else ranks):
            if self._get(self._key("left", r)) is not None:
                continue
            beat = self._get(self._key("beat", r))
            if beat is None:
                continue   # never joined
            if r != self.rank and now - float(beat) > self.timeout_s:
                continue   # silent for too long
            out.add(r)
        return out

    def departed(self) -> List[int]:
        return sorted(set(range(self.world)) - self.alive())

    def wait_for_all(self, timeout_s: float = 30.0) -> bool:
        """True once every rank has joined (used right after start-up)."""
        deadline = time.time() + timeout_s
        while time.time() < deadline:
            if len(self.alive()) == self.world:
                return True
            time.sleep(0.01)
        return False
