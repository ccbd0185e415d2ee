"""Rehearsal of the serial-versus-parallel convergence tooling on CPU ranks: generated configs, a tiny serial run and a
tiny 2-rank window-parallel run of ``train_scripts/test_pretrain.py`` (gloo), and the analysis report."""
import csv
import os
import subprocess
import sys
from pathlib import Path

import yaml

ROOT = Path(__file__).resolve().parents[1]
TOOLS = ROOT / "tests" / "distributed" / "correctness"


def _run(cmd, env, timeout=900):
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, f"{' '.join(map(str, cmd))}\n{p.stdout[-3000:]}\n{p.stderr[-3000:]}"
    return p


def test_generate_run_analyze(tmp_path):
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="",
               MODEL_PARALLEL_SIZE="2", DATA_PARALLEL_SIZE="1", CONFIG_DIR=str(tmp_path / "configs"),
               HEIGHT="64", WIDTH="128", PADDED_SHAPE_H="64", PADDED_SHAPE_W="128", NUM_CHANNELS="8", PATCH_SIZE="2",
               WINDOW_SIZE="4", SMALL_NUM_LAYERS="2", SMALL_EMBEDDING_DIM="32", SMALL_NUM_HEADS="2", PRECISION="fp32",
               USE_FAKE_INPUT="1", WARMUP_STEPS="1", LOSS_FUNC="MSE", NUM_WORKERS="0",
               SAMPLING_CHECKPOINT_DOWN="none", SAMPLING_CHECKPOINT_UP="none", ACTIVATION_MODE="none",
               MASTER_ADDR="127.0.0.1")
    _run([sys.executable, str(TOOLS / "generate_configs.py")], env)
    names = sorted(p.name for p in (tmp_path / "configs").iterdir())
    assert names == ["correctness_seq_fsdp.yaml", "correctness_topo_wp.yaml", "correctness_topo_wp_sp.yaml",
                     "correctness_topo_wp_tp.yaml"]
    wp = yaml.safe_load((tmp_path / "configs" / "correctness_topo_wp.yaml").read_text())
    assert wp["wp_topo"] == "(2, 1)" and wp["xfmr_wp_topo"] == "(2, 1)" and wp["model_type"] == "parallel"
    sp = yaml.safe_load((tmp_path / "configs" / "correctness_topo_wp_sp.yaml").read_text())
    assert sp["xfmr_wp_topo"] == "(1, 1)" and sp["xfmr_sp_size"] == 2 and sp["topology_label"] == "Topo(1,1,2,1)"

    results = tmp_path / "results"
    for case, nproc, port in (("seq_fsdp", 1, 29811), ("topo_wp", 2, 29812)):
        out = results / case
        out.mkdir(parents=True)
        cfg = tmp_path / "configs" / f"correctness_{case}.yaml"
        c = yaml.safe_load(cfg.read_text())
        c.update(fake_length=4, use_splited_data=(case != "seq_fsdp"))        # optimizer_config stays the generated 7 (sharded parameters)
        assert c["optimizer_config"] == 7
        cfg.write_text(yaml.safe_dump(c, sort_keys=False))
        _run([sys.executable, "-m", "torch.distributed.run", "--master_addr", "127.0.0.1", "--master_port", str(port),
              "--nnodes", "1", "--nproc_per_node", str(nproc), "train_scripts/test_pretrain.py",
              "--data_parallel_group_size", "1", "--model_cfg", str(cfg), "--steps", "3",
              "--metrics_csv", str(out / "loss.csv"), "--metrics_no_json", "--disable_rank_log_redirect",
              "--disable_torch_prof"], env)
        (out / "status.ok").write_text("done\n")
        assert len(list(csv.DictReader(open(out / "loss.csv")))) == 3

    p = subprocess.run([sys.executable, str(TOOLS / "analyze_correctness.py"), "--result_dir", str(results),
                        "--config_dir", str(tmp_path / "configs"), "--tolerance", "1e-3"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    rows = {r["case"]: r for r in csv.DictReader(open(results / "summary.csv"))}
    assert set(rows) == {"seq_fsdp", "topo_wp"}
    assert float(rows["topo_wp"]["max_abs_diff"]) <= 1e-3          # fp32, same seeds: the layouts agree
    assert "Activation settings identical across cases: yes" in (results / "report.md").read_text()
