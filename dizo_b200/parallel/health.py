"""Host-side failure detection: heartbeats through the rendezvous store.

Each rank writes ``(step, wall time)`` under its own key after every step and, before it
launches the next one, reads its peers' keys; a peer whose heartbeat is older than
``stale_after`` seconds (or that is more than ``max_lag`` steps behind) raises
:class:`PeerLost` on the host, before any kernel or collective that would wait for that peer is
launched.  ``sync(step)`` is the strict form the trainer uses: report, then wait on the host until
every peer has reported the same step (a store poll, about a millisecond per step), so a rank
that left between two steps is noticed before the step's first collective instead of inside it.
The reference has no failure detection at all (its only signal handling is the
SIGUSR1 callback, large_models/utils.py:291-315).
"""
from __future__ import annotations

import time


class PeerLost(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, store, rank: int, world: int, stale_after: float = 60.0, max_lag: int | None = None,
                 prefix: str = "dizo_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.stale_after, self.max_lag, self.prefix = stale_after, max_lag, prefix
        self._t_start = time.time()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def peers(self) -> dict[int, tuple[int, float]]:
        """Last (step, time) of every peer; (-1, 0.0) for a peer that has never reported.  The key is
        probed with ``store.check`` first: ``store.get`` of a missing key blocks until the store's own
        timeout (minutes), which would hide a rank that died before its first heartbeat."""
        out = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if not self.store.check([self._key(r)]):
                    out[r] = (-1, 0.0)
                    continue
                raw = self.store.get(self._key(r)).decode()
                s, t = raw.split(":")
                out[r] = (int(s), float(t))
            except Exception:
                out[r] = (-1, 0.0)
        return out

    def check(self, step: int) -> None:
        now = time.time()
        for r, (s, t) in self.peers().items():
            if s < 0:
                t = self._t_start            # never reported: silent since this monitor started
            if now - t > self.stale_after:
                raise PeerLost(f"rank {r} has not reported for {now - t:.1f}s (last step {s})")
            if self.max_lag is not None and step - s > self.max_lag:
                raise PeerLost(f"rank {r} is {step - s} steps behind")

    def sync(self, step: int, poll: float = 0.001) -> None:
        """Report ``step`` and wait (on the host) until every peer has reported it too."""
        self.beat(step)
        t0 = time.time()
        while True:
            behind = {r: s for r, (s, _) in self.peers().items() if s < step}
            if not behind:
                return
            if time.time() - t0 > self.stale_after:
                r, s = next(iter(behind.items()))
                raise PeerLost(f"rank {r} did not reach step {step} within {self.stale_after:.1f}s "
                               f"(last reported step {s})")
            time.sleep(poll)
