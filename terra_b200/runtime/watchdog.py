"""Host-side failure detection (the reference has none: a dead rank there shows up as a hung collective).

Two pieces, both free of any device-side fault:

* ``RankMonitor``: every rank publishes a heartbeat ``(step, wall time)`` in a ``torch.distributed`` store between
  steps; before launching the next step a rank asks for the peers that have stopped beating and raises
  ``PeerLost`` instead of entering a collective that would never complete.
* ``check_device_status``: turns the status word that the kernels' bounded waits write (mbarrier waits of the GEMM,
  waits on a peer's flag in the NVLink kernels) into a Python exception.

Recovery is the checkpoint / ``ckpt_start`` path of the training scripts; elastic resizing is out of scope (as in the
reference)."""
from __future__ import annotations

import time
from typing import Dict, List, Optional


class PeerLost(RuntimeError):
    """Raised on the surviving ranks when a peer stopped publishing heartbeats."""

    def __init__(self, ranks: List[int], detail: str = ""):
        super().__init__(f"ranks {ranks} stopped responding{(': ' + detail) if detail else ''}")
        self.ranks = ranks


class RankMonitor:
    def __init__(self, store, rank: int, world: int, stale_after_s: float = 60.0, prefix: str = "terra_hb", clock=time.time):
        self.store, self.rank, self.world = store, rank, world
        self.stale_after_s, self.prefix, self.clock = stale_after_s, prefix, clock
        self._last_seen: Dict[int, float] = {}

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        """Publish "alive at ``step``". Call between steps, with no kernel or collective of the step in flight."""
        self.store.set(self._key(self.rank), f"{step}:{self.clock():.3f}")

    def leave(self) -> None:
        """Announce an orderly exit so that the peers fail fast instead of waiting for the staleness limit."""
        self.store.set(self._key(self.rank), "left")

    def read(self, r: int) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return self.store.get(self._key(r)).decode()
        except Exception:
            return None

    def lost_peers(self, min_step: Optional[int] = None) -> List[int]:
        """Ranks that left, never showed up within the limit, or whose last beat is older than ``stale_after_s``
        (and, with ``min_step``, is from an earlier step than that)."""
        now, lost = self.clock(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self.read(r)
            if v == "left":
                lost.append(r)
                continue
            if v is None:
                first = self._last_seen.setdefault(r, now)
                if now - first > self.stale_after_s:
                    lost.append(r)
                continue
            step_s, t_s = v.split(":")
            self._last_seen[r] = float(t_s)
            if now - float(t_s) > self.stale_after_s and (min_step is None or int(step_s) < min_step):
                lost.append(r)
        return lost

    def assert_alive(self, min_step: Optional[int] = None) -> None:
        lost = self.lost_peers(min_step)
        if lost:
            raise PeerLost(lost)


def check_device_status(device) -> None:
    """Raise if a kernel's bounded wait ran out since the last check (synchronises the device)."""
    from ..ops.gemm import check_status

    check_status(device)
