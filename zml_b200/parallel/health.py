"""Host-side liveness of the ranks of a job: heartbeats through the rendezvous store.

In-kernel collectives make a rank's progress depend on its peers, so a rank that died must be
noticed on the host *before* the next launch (the kernels' bounded waits are the second line
of defence).  Every rank bumps a counter in the store between steps; `check()` raises
`RankFailure` naming the ranks whose counter has not moved for `timeout_s`, or that announced
an orderly exit with `leave()`.

The reference has no failure detection: a failed PJRT execute is a panic (zml/exe.zig:326-328).
"""
from __future__ import annotations

import time
from typing import Optional


class RankFailure(RuntimeError):
    def __init__(self, ranks, reason: str):
        super().__init__(f"rank(s) {sorted(ranks)} {reason}")
        self.ranks = sorted(ranks)
        self.reason = reason


class Heartbeat:
    """`store` is a torch.distributed store (TCPStore / FileStore / HashStore) shared by all ranks."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 10.0, prefix: str = "zb/hb"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = timeout_s
        self.prefix = prefix
        self._last_seen: dict[int, tuple[int, float]] = {}
        self.beat()

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self) -> int:
        """Call between steps, with no kernel or collective of this rank in flight."""
        return int(self.store.add(self._key(self.rank), 1))

    def leave(self) -> None:
        """Announces an orderly departure (the rank must not take part in later collectives)."""
        self.store.set(f"{self.prefix}/left/{self.rank}", b"1")

    def _count(self, rank: int) -> int:
        return int(self.store.add(self._key(rank), 0))

    def check(self, now: Optional[float] = None) -> None:
        """Raises RankFailure if a peer left or stopped beating; call before launching a step."""
        now = time.monotonic() if now is None else now
        left, silent = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check([f"{self.prefix}/left/{r}"]):
                left.append(r)
                continue
            c = self._count(r)
            seen = self._last_seen.get(r)
            if seen is None or c != seen[0]:
                self._last_seen[r] = (c, now)
            elif now - seen[1] > self.timeout_s:
                silent.append(r)
        if left:
            raise RankFailure(left, "left the job")
        if silent:
            raise RankFailure(silent, f"sent no heartbeat for {self.timeout_s} s")
