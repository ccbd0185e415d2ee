"""Checkpoint save -> resume round trips through the entry points themselves (CPU / gloo ranks):

* ``train.py`` on the serial model (``ckpt_layout: single``), on two window-parallel ranks with a replicated
  optimizer (``wp_rank``), with the sharded optimizer (``rank_local``) and with the reference's FSDP configurations
  (``fsdp_full``, ``fsdp_sharded``): two epochs in one run must give the same
  losses as one epoch, a save, and a second run that resumes from it;
* ``finetune.py``: step checkpoints (``save_interval_steps``) and resuming from ``ckpt_step``.

Reference behaviour: train_scripts/train.py:216-280, finetune.py:219-318.
"""
import os
import re
import socket
import subprocess
import sys

import pytest
import torch
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(script, cfg, tmp_path, name, nproc=1):
    path = tmp_path / f"{name}.yaml"
    path.write_text(yaml.safe_dump(cfg))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", PYTHONPATH=ROOT)
    exe = os.path.join(ROOT, "train_scripts", script)
    if nproc == 1:
        cmd = [sys.executable, exe, "--model_cfg", str(path)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
               "127.0.0.1", "--master-port", str(_free_port()), exe, "--model_cfg", str(path)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900, cwd=str(tmp_path))
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-4000:])


def _losses(log_path):
    """``[(global_step, loss)]`` of a rank-0 log file."""
    return [(int(g), float(v)) for v, g in re.findall(r"loss ([0-9.eE+-]+) lr: \S+ train_gs (\d+)", open(log_path).read())]


def _base(name, tmp_path, run):
    cfg = yaml.safe_load(open(os.path.join(ROOT, "configs", "model", "correctness", name)))
    cfg.update(train_path=str(tmp_path / run), max_train_steps_per_epoch=2, save_interval_epochs=1, fake_length=4,
               precision="fp32", warmup_steps=1)
    return cfg


@pytest.mark.parametrize("name,nproc,opt,layout", [
    ("tiny_seq_cpu.yaml", 1, 4, "single"),
    ("tiny_para_wp2.yaml", 2, 4, "wp_rank"),
    ("tiny_para_wp2.yaml", 2, 6, "rank_local"),
    ("tiny_para_wp2.yaml", 2, 7, "fsdp_full"),           # the reference's FSDP configurations: one gathered file ...
    ("tiny_para_wp2.yaml", 2, 7, "fsdp_sharded"),        # ... or every rank's own ranges of masters and moments
])
def test_pretrain_resume_matches_uninterrupted_run(tmp_path, name, nproc, opt, layout):
    extra = {"fsdp_checkpoint_type": layout[len("fsdp_"):]} if layout.startswith("fsdp_") else {}
    whole = dict(_base(name, tmp_path, "whole"), optimizer_config=opt, num_pre_train_epochs=2, **extra)
    _run("train.py", whole, tmp_path, "whole", nproc)
    first = dict(_base(name, tmp_path, "parts"), optimizer_config=opt, num_pre_train_epochs=1, **extra)
    _run("train.py", first, tmp_path, "first", nproc)
    # the cosine schedule depends on the planned number of epochs: keep it equal to the uninterrupted run's
    first_log = os.path.join(first["train_path"], first["description"], "loss", "rank0.txt")
    assert len(_losses(first_log)) == 2
    d = os.path.join(first["train_path"], first["description"], "ckpt")
    sub = {"single": "", "wp_rank": "wp_rank_0", "rank_local": "rank_0", "fsdp_full": "",
           "fsdp_sharded": os.path.join("fsdp_sharded", "rank_0")}[layout]
    blob = torch.load(os.path.join(d, sub, "epoch0.pth"), map_location="cpu", weights_only=False)
    assert blob["ckpt_layout"] == layout and blob["epoch"] == 0 and blob["global_step"] == 2
    assert set(blob) >= {"model_state_dict", "optimizer_state_dict", "loss", "epoch", "global_step", "ckpt_layout"}
    if layout == "fsdp_full":
        # one file, optimizer state in torch.optim.AdamW's per-parameter layout with whole-parameter tensors
        st = blob["optimizer_state_dict"]["state"]
        shapes = [tuple(v.shape) for v in blob["model_state_dict"].values()]
        assert all(tuple(e["exp_avg"].shape) in shapes for e in st.values()) and len(st) > 10
        assert not os.path.exists(os.path.join(d, "rank_1")) and not os.path.exists(os.path.join(d, "fsdp_sharded"))
    elif layout == "fsdp_sharded":
        ranges = blob["model_state_dict"]["__flat_ranges__"]
        owned = sum(r["hi"] - r["lo"] for r in ranges)
        assert 0 < owned < blob["model_state_dict"]["__numel__"], "a rank's file holds only the ranges it owns"
        assert os.path.exists(os.path.join(d, "fsdp_sharded", "rank_1", "epoch0.pth"))
    elif layout != "single":
        other = {"wp_rank": "wp_rank_1", "rank_local": "rank_1"}[layout]
        assert os.path.exists(os.path.join(d, other, "epoch0.pth")), "every owner rank writes its own file"
    second = dict(first, num_pre_train_epochs=2, ckpt_start=True, ckpt_epoch=0)
    _run("train.py", second, tmp_path, "second", nproc)
    resumed = _losses(first_log)                      # the log is appended to
    straight = _losses(os.path.join(whole["train_path"], whole["description"], "loss", "rank0.txt"))
    assert [g for g, _ in resumed] == [1, 2, 3, 4] == [g for g, _ in straight]
    # epoch 1 after the resume continues the optimizer state and the step counter: same losses as without the break
    # (steps 3, 4; steps 1, 2 differ only through the learning-rate horizon of the shorter first run)
    for (_, a), (_, b) in zip(resumed[2:], straight[2:]):
        assert abs(a - b) <= 2e-4 * abs(b), (resumed, straight)


@pytest.mark.parametrize("opt,kind,sub", [(4, "single", ""), (7, "fsdp_sharded", os.path.join("fsdp_sharded", "rank_0"))])
def test_finetune_step_checkpoint_and_resume(tmp_path, opt, kind, sub):
    """The rollout loop saves every ``save_interval_steps`` steps; resuming from such a file continues inside the epoch:
    the steps already taken are skipped and the next one reproduces the uninterrupted run's loss (replicated parameters,
    and sharded parameters with per-rank files)."""
    cfg = yaml.safe_load(open(os.path.join(ROOT, "configs", "finetuning", "tiny_finetune_seq.yaml")))
    cfg.update(train_path=str(tmp_path / "ft"), max_train_steps_per_epoch=3, save_interval_steps=2, precision="fp32",
               finetune_lead_time=2, num_finetune_epochs=1, fake_length=4, optimizer_config=opt,
               fsdp_checkpoint_type="sharded")
    cfg.pop("activation", None)
    _run("finetune.py", cfg, tmp_path, "ft1")
    base = os.path.join(cfg["train_path"], cfg["description"], "lead_2")
    assert os.path.exists(os.path.join(base, "ckpt", sub, "step2.pth")) and os.path.exists(os.path.join(base, "ckpt", sub, "epoch0.pth"))
    blob = torch.load(os.path.join(base, "ckpt", sub, "step2.pth"), map_location="cpu", weights_only=False)
    assert blob["global_step"] == 2 and blob["ckpt_layout"] == kind
    log = os.path.join(base, "loss", "rank0.txt")
    before = open(log).read().strip().splitlines()
    assert len(before) == 3 and "finetune step: 2 " in before[-1]
    _run("finetune.py", dict(cfg, ckpt_start=True, ckpt_step=2, ckpt_epoch=None), tmp_path, "ft2")
    lines = open(log).read().strip().splitlines()
    assert len(lines) == len(before) + 1, "steps 0 and 1 of the epoch are skipped, step 2 runs"
    assert "train_gs 2 " in lines[-1] and "finetune step: 2 " in lines[-1], lines[-1]     # counters from the checkpoint
    loss = lambda line: float(re.search(r"loss ([0-9.eE+-]+) lr:", line).group(1))
    assert abs(loss(lines[-1]) - loss(before[-1])) <= 1e-6 * abs(loss(before[-1])), (lines[-1], before[-1])


def test_finetune_harness_data_path_switches(tmp_path):
    """``test_finetune.py`` with the reference's data-path keys: a blocking single upload instead of the double buffer,
    the upload counted into the step time, the CPU batch released after the transfer; per-lead plans applied; and the
    combination the reference refuses (double buffering with blocking copies) refused here too."""
    import csv

    cfg = yaml.safe_load(open(os.path.join(ROOT, "configs", "finetuning", "tiny_finetune_seq.yaml")))
    cfg.update(train_path=str(tmp_path / "ft"), precision="fp32", finetune_lead_time=2, fake_length=3,
               input_double_buffer=False, input_transfer_non_blocking=False, include_input_transfer_in_step_time=True,
               release_cpu_batch_after_transfer=True)
    path = tmp_path / "ok.yaml"
    path.write_text(yaml.safe_dump(cfg))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", PYTHONPATH=ROOT)
    exe = os.path.join(ROOT, "train_scripts", "test_finetune.py")
    out = subprocess.run([sys.executable, exe, "--model_cfg", str(path), "--steps", "2", "--metrics_csv",
                          str(tmp_path / "m.csv"), "--memory_timeline_csv", str(tmp_path / "leads.csv"), "--metrics_no_json",
                          "--disable_torch_prof", "--disable_rank_log_redirect"], env=env, capture_output=True, text=True,
                         timeout=900, cwd=str(tmp_path))
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-4000:])
    rows = list(csv.DictReader(open(tmp_path / "m.csv")))
    assert len(rows) == 2 and all(float(r["input_transfer_time_s"]) > 0 for r in rows)
    assert all(float(r["step_time_s"]) > float(r["input_transfer_time_s"]) for r in rows)
    leads = list(csv.DictReader(open(tmp_path / "leads.csv")))
    assert [int(r["lead"]) for r in leads] == [1, 2, 1, 2]            # two leads per step, numbered from 1
    assert [r["checkpoint_layers"] for r in leads[:2]] == ["[]", '["0-1"]'] and leads[1]["checkpoint_label"] == "lead2-2"
    assert {r["transformer_activation_mode"] for r in leads} == {"none", "torch_recompute"}

    # pretrained weights named by the config are imported before the run (here: every tensor zeroed, so the first loss
    # is that of a model that outputs its bias-free zero field and differs from the seeded initialisation's)
    maker = ("import sys, torch; sys.path.insert(0, %r); from train_scripts.common import FINETUNE_DEFAULTS, Session; "
             "s = Session(%r, 1, dict(FINETUNE_DEFAULTS, use_fake_input=True)); "
             "torch.save({'model_state_dict': {k: torch.zeros_like(v) for k, v in s.model.state_dict().items()}}, %r); s.close()"
             % (ROOT, str(path), str(tmp_path / "zero.pth")))
    made = subprocess.run([sys.executable, "-c", maker], env=env, capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert made.returncode == 0, made.stderr[-3000:]
    path3 = tmp_path / "pre.yaml"
    path3.write_text(yaml.safe_dump(dict(cfg, trained_model_checkpoint_path=str(tmp_path / "zero.pth"))))
    out = subprocess.run([sys.executable, exe, "--model_cfg", str(path3), "--steps", "1", "--metrics_csv",
                          str(tmp_path / "pre.csv"), "--metrics_no_json", "--disable_torch_prof", "--disable_rank_log_redirect"],
                         env=env, capture_output=True, text=True, timeout=900, cwd=str(tmp_path))
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-4000:])
    assert "[pretrained] loaded" in out.stdout and "No trained_model_config_path" not in out.stdout
    first = list(csv.DictReader(open(tmp_path / "pre.csv")))[0]
    assert abs(float(first["loss"]) - float(rows[0]["loss"])) > 1e-3 * float(rows[0]["loss"])

    bad = dict(cfg, input_double_buffer=True)
    path2 = tmp_path / "bad.yaml"
    path2.write_text(yaml.safe_dump(bad))
    out = subprocess.run([sys.executable, exe, "--model_cfg", str(path2), "--steps", "1", "--metrics_no_json",
                          "--disable_torch_prof", "--disable_rank_log_redirect"], env=env, capture_output=True, text=True,
                         timeout=900, cwd=str(tmp_path))
    assert out.returncode != 0 and "input_double_buffer requires input_transfer_non_blocking=true" in out.stderr
