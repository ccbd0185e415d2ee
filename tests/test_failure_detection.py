"""Failure detection without any GPU fault: heartbeats in a store, a rank that leaves between steps (gloo CPU ranks),
and, on a GPU, a bounded device-side wait that runs out and reports through the status word."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_rank_monitor_detects_stale_and_left_peers():
    import torch.distributed as dist

    from terra_b200.runtime.watchdog import PeerLost, RankMonitor

    store = dist.HashStore()
    now = [1000.0]
    mons = [RankMonitor(store, r, 3, stale_after_s=5.0, clock=lambda: now[0]) for r in range(3)]
    for m in mons:
        m.beat(0)
    assert mons[0].lost_peers() == []
    now[0] += 4.0
    mons[0].beat(1)
    mons[1].beat(1)            # rank 2 stops beating
    now[0] += 4.0
    assert mons[0].lost_peers(min_step=1) == [2]
    with pytest.raises(PeerLost) as e:
        mons[1].assert_alive(min_step=1)
    assert e.value.ranks == [2]
    mons[1].leave()            # an orderly exit is seen at once
    assert mons[0].lost_peers() == [1, 2]


def test_rank_that_finished_the_same_step_and_left_is_not_a_failure():
    """Ranks end a run at slightly different times: a peer that left after completing step s is lost only to a rank
    that expects it at a later step."""
    import torch.distributed as dist

    from terra_b200.runtime.watchdog import RankMonitor

    store = dist.HashStore()
    a, b = RankMonitor(store, 0, 2, stale_after_s=60.0), RankMonitor(store, 1, 2, stale_after_s=60.0)
    a.beat(3)
    b.beat(3)
    b.leave()                                   # rank 1 finished its last step (3) and exits
    assert a.lost_peers(min_step=3) == []       # rank 0 is still wrapping up step 3: fine
    assert a.lost_peers(min_step=4) == [1]      # it would be missing from step 4
    assert a.lost_peers() == [1]


def test_rank_that_never_joins_is_reported_after_the_limit():
    import torch.distributed as dist

    from terra_b200.runtime.watchdog import RankMonitor

    now = [0.0]
    m = RankMonitor(dist.HashStore(), 0, 2, stale_after_s=3.0, clock=lambda: now[0])
    m.beat(0)
    assert m.lost_peers() == []
    now[0] = 2.0
    assert m.lost_peers() == []
    now[0] = 4.0
    assert m.lost_peers() == [1]


WORKER = textwrap.dedent("""
    import datetime, os, sys, time
    import torch, torch.distributed as dist
    from terra_b200.runtime.watchdog import PeerLost, RankMonitor
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method="env://", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    store = dist.distributed_c10d._get_default_store()
    mon = RankMonitor(store, rank, world, stale_after_s=30.0)
    x = torch.ones(4)
    for step in range(3):
        mon.beat(step)
        if rank == 1 and step == 1:
            mon.leave()                     # leaves between steps, nothing of its own in flight
            print("rank1 left", flush=True)
            os._exit(0)
        # the survivors learn of it on the host before their next collective
        time.sleep(0.5 if step == 1 else 0.0)
        try:
            mon.assert_alive()
        except PeerLost as e:
            print(f"rank{rank} detected {e.ranks} before step {step}", flush=True)
            os._exit(0)
        dist.all_reduce(x)
    print(f"rank{rank} finished without detection", flush=True)
    os._exit(1)
""")


def test_rank_leaving_between_steps_is_detected_on_the_host(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes", "1", "--nproc_per_node", "3",
                        "--master_addr", "127.0.0.1", "--master_port", "29841", str(script)],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    out = p.stdout + p.stderr
    assert "rank1 left" in out
    assert "rank0 detected [1] before step 1" in out and "rank2 detected [1] before step 1" in out, out[-3000:]
    assert "finished without detection" not in out


@pytest.mark.gpu
def test_bounded_peer_wait_reports_through_the_status_word():
    """A barrier whose second participant never signals: the device-side wait gives up after its time budget, the
    kernel returns, the host raises, and the context is still usable afterwards."""
    from terra_b200 import _ext
    from terra_b200.ops.gemm import check_status, status_word

    ext = _ext.load()
    pads = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]   # "peer 1" is a buffer nobody drives
    st = status_word("cuda")
    st.zero_()
    ext.peer_barrier([p.data_ptr() for p in pads], 0, 1, st, int(50e6))            # 50 ms budget
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="error 2"):
        check_status("cuda")
    # the context survived: a normal kernel still runs and the status word is clean again
    a = torch.ones(8, device="cuda")
    assert float((a * 2).sum().item()) == 16.0
    check_status("cuda")


def test_step_guard_raises_on_a_lost_peer_and_releases_the_arenas():
    """What the training loops call between steps: a peer that stopped beating turns into ``PeerLost`` on the host,
    and every arena's stream waits are released first so that nothing of this process stays blocked on the dead peer."""
    import torch.distributed as dist

    from terra_b200.runtime.watchdog import PeerLost, RankMonitor, StepGuard

    class FakeArena:
        released = 0

        def release_waits(self):
            FakeArena.released += 1

    store = dist.HashStore()
    now = [0.0]
    mons = [RankMonitor(store, r, 2, stale_after_s=5.0, clock=lambda: now[0]) for r in range(2)]
    guard = StepGuard("cpu", mons[0], arenas=[FakeArena(), FakeArena()])
    mons[1].beat(0)
    guard.after_step(0)                       # both alive
    now[0] = 10.0                             # rank 1 never beats again
    with pytest.raises(PeerLost) as e:
        guard.after_step(1)
    assert e.value.ranks == [1] and FakeArena.released == 2


def test_training_loop_raises_when_a_watchdog_released_a_wait():
    from terra_b200.runtime.watchdog import StepGuard, StreamWaitExpired

    class Tripped:
        def check(self):
            raise StreamWaitExpired("released")

        def close(self):
            pass

    guard = StepGuard("cpu", None, watchdogs=[Tripped()])
    with pytest.raises(StreamWaitExpired):
        guard.after_step(0)


@pytest.mark.gpu
def test_stream_wait_on_a_silent_peer_is_released_by_the_host_watchdog():
    """The copy-engine all-gather waits for a peer's signal with a stream memory operation, which has no time limit.
    Here a side stream waits on a word that nobody ever writes (the host-made failure: the "peer" simply does not
    publish); the watchdog releases the wait after its budget, the stream drains, the event is reported - and no kernel
    ever spun on the GPU."""
    import time

    from terra_b200 import _ext
    from terra_b200.runtime.watchdog import StreamWaitExpired, StreamWaitWatchdog

    ext = _ext.load()
    words = torch.zeros(16, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    side = torch.cuda.Stream()

    class Arena:
        buf = words

        def release_waits(self):
            s = torch.cuda.Stream()
            for i in range(16):
                ext.stream_write_value(s.cuda_stream, words.data_ptr() + 4 * i, 0x7F7F7F7F)
            s.synchronize()

    wd = StreamWaitWatchdog(Arena(), lambda: side, budget_s=0.3, poll_s=0.02)
    ext.stream_wait_value(side.cuda_stream, words.data_ptr() + 4 * 3, 1)      # waits for word 3 >= 1: never written
    marker = torch.zeros(1, device="cuda")
    with torch.cuda.stream(side):
        marker += 1                                                             # queued behind the wait
    wd.arm()
    t0 = time.time()
    while not side.query() and time.time() - t0 < 10.0:
        time.sleep(0.02)
    assert side.query(), "the side stream is still blocked"
    assert 0.2 < time.time() - t0 < 5.0
    torch.cuda.synchronize()
    assert float(marker.item()) == 1.0
    with pytest.raises(StreamWaitExpired):
        wd.check()
    wd.check()                                # reported once
    wd.close()
    # main stream and context are fine
    assert float((torch.ones(4, device="cuda") * 3).sum().item()) == 12.0
