"""Parameter sharding (the FSDP / ZeRO-3 role) on gloo CPU ranks: the schedule of gathers and releases, the sharded
optimizer against ``torch.optim.AdamW``, both checkpoint forms, and the framework's configurations 5 / 7 / 9 against its
sharded optimizer (configuration 6) on the same model and data."""
import csv
import json
import os
import socket
import subprocess
import sys

import pytest
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _torchrun(nproc, script, *args, timeout=900):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes", "1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", str(_port()), script, *args]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-5000:])
    return p.stdout


@pytest.mark.parametrize("nproc,mode", [
    (2, {}),
    (2, {"recompute": True, "prefetch": "overlap"}),
    (2, {"rollout": 2, "clip": True}),
    (2, {"whole_model": True}),
    (3, {"recompute": True, "blocks_per_unit": 2}),
    (3, {"prefetch": "overlap", "rollout": 2}),
    (2, {"reshard_after_forward": False, "recompute": True}),
])
def test_sharded_parameters_train_like_adamw_on_the_summed_loss(nproc, mode):
    out = _torchrun(nproc, os.path.join(ROOT, "tests", "param_sharding_worker.py"), json.dumps(mode), timeout=600)
    res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    passes = mode.get("rollout", 1)
    # per unit and step: one gather for each forward pass and one for each backward pass through it, never two (a
    # recomputed segment stays resident for its backward pass; a prefetched unit is not gathered again); the root
    # unit is gathered once per step. 5 training steps and one evaluation ran.
    blocks, root = res["gathers"][:-1], res["gathers"][-1]
    if mode.get("reshard_after_forward", True):
        assert root == 6 and all(g == 5 * 2 * passes + passes for g in blocks), res
    else:
        # kept between forward and backward: one gather per training step (the evaluation pass gathers once more)
        assert root == 6 and all(g == 6 for g in blocks), res
    assert all(r == 5 * passes for r in res["reductions"][:-1]) and res["reductions"][-1] == 5
    # the gradient observer (the DEBUG_GRAD_HOOK report of sharded parameters) ran once per reduction, with one line per
    # parameter that had a gradient
    assert res["observed"] == sum(res["reductions"]) and res["lines"] >= res["observed"], res
    assert res["first_line"].startswith("[grad hook] "), res
    if not mode.get("whole_model") and not mode.get("recompute"):
        # values and gradients of at most two units (the running one and a prefetched neighbour) next to the root's
        assert res["peak_bytes"] < 2 * res["total_bytes"] * (0.5 if mode.get("prefetch") else 0.4), res


def test_working_copy_bookkeeping_of_the_gpu_form():
    """With a bf16 working copy (the GPU form, forced on CPU tensors here) that copy is what the units gather, the fp32
    values stay released outside ``summon_full_params``, the optimizer keeps the owned bf16 slices current, and the
    gathered model equals ``torch.optim.AdamW``'s."""
    out = _torchrun(2, os.path.join(ROOT, "tests", "param_sharding_worker.py"), json.dumps({"working_copy": True}), timeout=600)
    res = json.loads([l for l in out.splitlines() if l.startswith("RESULT ")][-1][len("RESULT "):])
    assert res["worst"] < 1e-6


def _pretrain_losses(tmp_path, tag, cfg, nproc, steps=4):
    path = tmp_path / f"{tag}.yaml"
    path.write_text(yaml.safe_dump(cfg, sort_keys=False))
    out = tmp_path / f"{tag}.csv"
    log = _torchrun(nproc, os.path.join(ROOT, "train_scripts", "test_pretrain.py"), "--model_cfg", str(path), "--steps",
                    str(steps), "--metrics_csv", str(out), "--metrics_no_json", "--disable_rank_log_redirect",
                    "--disable_torch_prof")
    return [float(r["loss"]) for r in csv.DictReader(open(out))], log


def test_fsdp_configurations_match_the_sharded_optimizer(tmp_path):
    """``optimizer_config`` 9 on a TP = 2 layout (TP shards stay with their TP rank, everything else is split over
    both ranks), with a recomputed segment and prefetching, and 5 / 7 on the WP = 2 layout: the same losses as
    configuration 6, whose gradient convention they share."""
    base = yaml.safe_load(open(os.path.join(ROOT, "configs", "model", "correctness", "tiny_para_wp2.yaml")))
    base.update(train_path=str(tmp_path / "out"), precision="fp32")
    tp = dict(base, xfmr_wp_topo="(1, 1)", tensor_parallel_size=2, window_assignment_mode="regular", num_heads=[4, 8],
              embedding_dim=128, activation=dict(mode="torch_recompute", checkpoint_layers=["0-1"]))
    want, _ = _pretrain_losses(tmp_path, "tp6", dict(tp, optimizer_config=6), 2)
    got, log = _pretrain_losses(tmp_path, "tp9", dict(tp, optimizer_config=9, FSDP_CONFIG7_PREFETCH_POLICY="overlap"), 2)
    assert "[FSDP] optimizer_config=9" in log and "group sizes=[1, 2]" in log and "prefetch_policy=overlap" in log
    assert want[-1] < want[0] and all(abs(a - b) <= 1e-6 * abs(b) for a, b in zip(got, want)), (got, want)

    # the sampling path as units of its own (bracketed function calls), with its checkpoint modes and prefetching
    act = dict(mode="torch_recompute", checkpoint_layers=["0-1", "D1", "U0"])
    want, _ = _pretrain_losses(tmp_path, "s6", dict(base, optimizer_config=6, activation=act), 2, steps=3)
    got, log = _pretrain_losses(tmp_path, "s7", dict(base, optimizer_config=7, activation=act, FSDP_SAMPLING_WRAPPER_CFG=1,
                                                     FSDP_CONFIG7_PREFETCH_POLICY="overlap"), 2, steps=3)
    assert "units=8 (+root=False)" in log and "sampling_wrapper_cfg=1" in log
    assert all(abs(a - b) <= 1e-6 * abs(b) for a, b in zip(got, want)), (got, want)

    want, _ = _pretrain_losses(tmp_path, "wp6", dict(base, optimizer_config=6), 2)
    for oc in (5, 7):
        got, log = _pretrain_losses(tmp_path, f"wp{oc}", dict(base, optimizer_config=oc), 2)
        assert f"[FSDP] optimizer_config={oc}" in log and ("units=0" in log) == (oc == 5)
        assert all(abs(a - b) <= 1e-6 * abs(b) for a, b in zip(got, want)), (oc, got, want)


def test_fsdp_configurations_keep_the_reference_preconditions():
    """5 / 7 are refused with tensor parallelism and 8 / 9 without it, in the reference's words."""
    import torch

    from terra_b200.models.get_model import get_model_for_train

    for oc, tp, text in ((7, 2, "only allowed when tensor_parallel_size == 1"), (5, 2, "only allowed when"),
                         (9, 1, "requires tensor_parallel_size > 1"), (8, 1, "requires tensor_parallel_size > 1")):
        with pytest.raises(ValueError, match=text):
            get_model_for_train({"model_architecture": "none"}, {"optimizer_config": oc, "tensor_parallel_size": tp})
