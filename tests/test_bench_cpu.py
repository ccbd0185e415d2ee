"""The benchmark harness rehearsed on two gloo CPU ranks with the smoke model: one JSON line, the factorised extra
layout timed in child processes with a rendezvous of their own, and a headline that survives a child that does not
answer in time."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _bench(tmp_path, *extra):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", PYTHONPATH=ROOT, TERRA_NUMA_BIND="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "bench.py"), "--gpus", "2", "--small", "--steps", "1",
           "--warmup", "1", *extra]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=str(tmp_path))
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-4000:])
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, lines                     # rank 0 prints exactly one JSON line
    return json.loads(lines[0])


def test_bench_line_with_extra_layout_from_child_processes(tmp_path):
    line = _bench(tmp_path, "--extra-layout", "1,2,1", "--extra-deadline", "400")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["e2e"]["h2d_bytes_per_step"] > 0
    extra = line["layout_1x2x1"]
    assert "error" not in extra, extra
    assert extra["layout"] == "wg1xsp2xtp1" and extra["ms_per_step"] > 0 and abs(extra["loss"] - line["loss"]) < 0.05


def test_bench_headline_survives_a_child_that_misses_the_deadline(tmp_path):
    line = _bench(tmp_path, "--extra-layout", "1,2,1", "--extra-deadline", "0.5")
    assert line["value"] > 0 and "no result within" in line["layout_1x2x1"]["error"]
