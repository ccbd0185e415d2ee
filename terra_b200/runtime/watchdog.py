"""Host-side failure detection (the reference has none: a dead rank there shows up as a hung collective).

Pieces, all free of any device-side fault:

* ``RankMonitor``: every rank publishes a heartbeat ``(step, wall time)`` in a ``torch.distributed`` store between
  steps; before launching the next step a rank asks for the peers that have stopped beating and raises
  ``PeerLost`` instead of entering a collective that would never complete.
* ``check_device_status``: turns the status word that the kernels' bounded waits write (mbarrier waits of the GEMM,
  waits on a peer's flag in the NVLink kernels) into a Python exception.

* ``StreamWaitWatchdog``: a host thread that bounds the stream memory-operation waits of the copy-engine all-gather
  (they have no time limit of their own): past the budget it releases the waits and records the failure.
* ``StepGuard``: what the training loops call between steps - heartbeat, peer check, status word, watchdogs; on a
  lost peer it releases every arena's stream waits before raising.

Recovery is the checkpoint / ``ckpt_start`` path of the training scripts; elastic resizing is out of scope (as in the
reference)."""
from __future__ import annotations

import os
import threading
import time
from typing import Callable, Dict, List, Optional


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
        self._last_step = int(step)
        self.store.set(self._key(self.rank), f"{step}:{self.clock():.3f}")

    def leave(self) -> None:
        """Announce an orderly exit so that the peers fail fast instead of waiting for the staleness limit. The last
        step this rank completed goes with it: a peer that is still finishing that same step (ranks end a run at
        slightly different times) must not take the exit for a failure."""
        self.store.set(self._key(self.rank), f"left:{getattr(self, '_last_step', -1)}")

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
            if v is not None and v.startswith("left"):
                left_after = int(v.split(":")[1]) if ":" in v else -1
                if min_step is None or left_after < min_step:
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


class StreamWaitExpired(RuntimeError):
    """A stream memory-operation wait on a peer's signal outlived its budget and was released by the host."""


class StreamWaitWatchdog:
    """Bounds the waits that ``gather_shards_async`` queues on a side stream. ``arm()`` (called when a gather is queued)
    sets a deadline ``budget_s`` ahead; a daemon thread polls the stream and, if it is still busy past the deadline,
    calls ``arena.release_waits()`` - the queued waits complete, the stream drains, nothing is left blocked - and
    remembers the event. ``check()`` (training loop, between steps) raises it. The gathered data of a released wait is
    incomplete, so the step's result must be discarded: the loop stops and resumes from the last checkpoint."""

    def __init__(self, arena, stream_of: Callable[[], object], budget_s: Optional[float] = None, poll_s: float = 0.05):
        self.arena, self.stream_of = arena, stream_of
        self.budget_s = float(os.environ.get("TERRA_PEER_WAIT_MS", "5000")) * 1e-3 if budget_s is None else budget_s
        self.poll_s = poll_s
        self.tripped: Optional[str] = None
        self._deadline: Optional[float] = None
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._stop = False

    def arm(self) -> None:
        with self._lock:
            self._deadline = time.monotonic() + self.budget_s
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="terra-stream-wait-watchdog", daemon=True)
            self._thread.start()

    def _run(self) -> None:
        import torch

        dev = getattr(getattr(self.arena, "buf", None), "device", None)
        if dev is not None and dev.type == "cuda":
            torch.cuda.set_device(dev)
        while not self._stop:
            time.sleep(self.poll_s)
            with self._lock:
                deadline = self._deadline
            if deadline is None:
                continue
            stream = self.stream_of()
            if stream is None or stream.query():        # drained: every wait was satisfied
                with self._lock:
                    if self._deadline == deadline:
                        self._deadline = None
                continue
            if time.monotonic() > deadline:
                self.tripped = (f"a stream wait on a peer's signal was still pending {self.budget_s:.2f} s after it was "
                                "queued; released by the host watchdog")
                try:
                    self.arena.release_waits()
                finally:
                    with self._lock:
                        self._deadline = None

    def check(self) -> None:
        if self.tripped is not None:
            msg, self.tripped = self.tripped, None
            raise StreamWaitExpired(msg)

    def close(self) -> None:
        self._stop = True


class StepGuard:
    """Failure detection wired into a training loop. Call ``after_step(step)`` once per step where the host already
    synchronises (after the loss was read): it raises ``RuntimeError`` when a kernel's bounded wait ran out (status
    word), ``StreamWaitExpired`` when a watchdog released a stream wait, and ``PeerLost`` when a peer stopped
    beating - in which case every symmetric arena's stream waits are released first, so that no stream of this
    process stays blocked on the dead peer."""

    def __init__(self, device, monitor: Optional[RankMonitor] = None, model=None, optimizer=None, arenas=(),
                 watchdogs=(), check_every: int = 1):
        self.device, self.monitor = device, monitor
        self.model, self.optimizer = model, optimizer
        self.extra_arenas, self.extra_watchdogs = list(arenas), list(watchdogs)
        self.check_every = max(1, int(check_every))

    def arenas(self):
        real = self.model.module if hasattr(self.model, "module") else self.model
        pctx = getattr(real, "pctx", None)
        found = [getattr(pctx, n, None) for n in ("attn_arena", "tp_arena", "dom_arena")]
        fused = getattr(self.optimizer, "fused", None)
        if fused is not None:
            found += list(getattr(fused, "arenas", {}).values())
        return [a for a in found if a is not None] + self.extra_arenas

    def watchdogs(self):
        real = self.model.module if hasattr(self.model, "module") else self.model
        tpc = getattr(getattr(real, "pctx", None), "tp_comm", None)
        wd = getattr(tpc, "watchdog", None)
        return ([wd] if wd is not None else []) + self.extra_watchdogs

    def after_step(self, step: int) -> None:
        import torch

        for w in self.watchdogs():
            w.check()
        if torch.device(self.device).type == "cuda" and step % self.check_every == 0:
            check_device_status(self.device)
        if self.monitor is not None:
            self.monitor.beat(step)
            try:
                self.monitor.assert_alive(min_step=step)
            except PeerLost:
                self.release()
                raise

    def release(self) -> None:
        for a in self.arenas():
            try:
                a.release_waits()
            except Exception:
                pass

    def close(self, announce: bool = True) -> None:
        """``announce``: tell the peers that this rank leaves (they then fail fast). Not wanted when only this guard's
        model is dropped and the process carries on with another one."""
        if self.monitor is not None and announce:
            try:
                self.monitor.leave()
            except Exception:
                pass
        for w in self.watchdogs():
            w.close()


_guards_made = 0


def make_step_guard(device, rank: int, world: int, model=None, optimizer=None) -> StepGuard:
    """The guard the entry points use: heartbeats go through the default process group's store
    (``TERRA_HEARTBEAT_STALE_S`` seconds without a beat, default 120, count as lost). Every guard of a process gets
    its own key prefix (all ranks build their guards in the same order), so a second trainer in the same job does not
    read the first one's last words."""
    import torch.distributed as dist

    global _guards_made
    monitor = None
    if world > 1 and dist.is_available() and dist.is_initialized():
        store = dist.distributed_c10d._get_default_store()
        monitor = RankMonitor(store, rank, world, stale_after_s=float(os.environ.get("TERRA_HEARTBEAT_STALE_S", "120")),
                              prefix=f"terra_hb{_guards_made}")
    _guards_made += 1
    return StepGuard(device, monitor, model, optimizer)
