"""Host-side failure detection for a rank group: heartbeats over the rendezvous store.

The reference has no failure handling beyond status returns (threading/linux.mojo:305-312 waits forever).  Here every
device-side wait is bounded and reports through a status word, and the *host* notices a peer that stopped making
progress: each rank bumps a counter in the shared key-value store from a background thread; ``dead_ranks`` lists the
ranks whose counter did not move for ``timeout_s``.  A serving loop calls ``check()`` between steps, before launching
the next collective, so that a missing peer turns into an exception on the host instead of a timed-out kernel.
Nothing here touches a GPU.
"""
from __future__ import annotations

import threading
import time


class RankFailure(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"ranks {sorted(ranks)} stopped sending heartbeats")
        self.ranks = sorted(ranks)


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 0.1, timeout_s: float = 1.0, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._last_seen: dict[int, tuple[int, float]] = {}
        self._beats = 0
        self._dead: list[int] = []          # filled by the monitor thread (``start(monitor=True)``)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def start(self, monitor: bool = False) -> "Heartbeat":
        """Begin beating.  With ``monitor`` the same thread also watches the peers, so that the serving loop's
        ``check_fast()`` between steps is a plain memory read instead of a round trip to the store per peer."""
        self.store.set(self._key(self.rank), "0")

        def loop():
            while not self._stop.wait(self.interval_s):
                self._beats += 1
                try:
                    self.store.set(self._key(self.rank), str(self._beats))
                except Exception:
                    return        # the store went away: peers will see us as dead, which is the truth
                if monitor:
                    try:
                        dead = self.dead_ranks()
                    except Exception:
                        dead = []
                    if dead:
                        self._dead = dead

        self._thread = threading.Thread(target=loop, name=f"heartbeat-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1.0)

    def dead_ranks(self) -> list[int]:
        """Ranks whose heartbeat has not advanced for ``timeout_s`` (a rank never seen at all counts from first look)."""
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if not self.store.check([self._key(r)]):
                    value = -1
                else:
                    value = int(self.store.get(self._key(r)))
            except Exception:
                value = -2
            prev = self._last_seen.get(r)
            if prev is None or prev[0] != value:
                self._last_seen[r] = (value, now)
            elif now - prev[1] > self.timeout_s:
                dead.append(r)
        return dead

    def check(self) -> None:
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead)

    def check_fast(self) -> None:
        """Raise if the monitor thread has declared a peer dead; costs no store traffic (call it between steps)."""
        if self._dead:
            raise RankFailure(self._dead)

    def wait_for_failure(self, max_wait_s: float) -> list[int]:
        """Poll until some rank is declared dead or ``max_wait_s`` passed; returns the dead ranks (possibly empty)."""
        t0 = time.monotonic()
        while time.monotonic() - t0 < max_wait_s:
            dead = self.dead_ranks()
            if dead:
                return dead
            time.sleep(self.interval_s)
        return []
