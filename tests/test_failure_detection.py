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
