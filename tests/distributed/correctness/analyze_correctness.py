#!/usr/bin/env python3
"""Compares the loss curves of the convergence experiment's cases against a baseline case (reference:
tests/distributed/correctness/analyze_correctness.py). Reads ``<result_dir>/<case>/loss.csv`` (columns ``iter``,
``loss``, optional ``step_time_s``, ``peak_memory_mb``) and the generated YAML of each case, checks that all cases
used the same activation settings, and writes

* ``summary.csv``  one row per case: steps, first / final loss, max and mean absolute loss difference to the baseline,
  the step of the largest difference, final-loss delta, median step time, peak memory;
* ``report.md``    the same as a table plus the verdict against ``--tolerance`` (no tolerance: informational);
* ``loss_curves.png`` / ``loss_delta.png`` when matplotlib is importable (headless ``Agg`` backend), else a
  ``loss_delta.csv`` with the per-step differences.

    python tests/distributed/correctness/analyze_correctness.py [--result_dir D] [--config_dir D] [--baseline seq_fsdp]
"""
from __future__ import annotations

import argparse
import csv
import statistics
import sys
from pathlib import Path

import yaml

HERE = Path(__file__).resolve().parent


def read_curve(path: Path):
    rows = []
    with open(path, newline="") as f:
        for r in csv.DictReader(f):
            def num(key, default=None):
                try:
                    return float(r[key])
                except (KeyError, TypeError, ValueError):
                    return default
            it = num("iter", num("step", len(rows)))
            loss = num("loss")
            if loss is None:
                continue
            rows.append({"iter": int(it), "loss": loss, "step_time_s": num("step_time_s"), "peak_memory_mb": num("peak_memory_mb")})
    return rows


def load_cases(result_dir: Path, config_dir: Path, wanted):
    out = {}
    for d in sorted(p for p in result_dir.iterdir() if p.is_dir()):
        if wanted and d.name not in wanted:
            continue
        curve = d / "loss.csv"
        if not curve.exists():
            continue
        cfg_path = config_dir / f"correctness_{d.name}.yaml"
        cfg = yaml.safe_load(cfg_path.read_text()) if cfg_path.exists() else {}
        out[d.name] = {"rows": read_curve(curve), "cfg": cfg or {}, "ok": (d / "status.ok").exists()}
    return out


def activation_mismatches(cases):
    """Cases must differ in layout only: the activation block has to be identical."""
    blocks = {name: yaml.safe_dump(c["cfg"].get("activation", {}), sort_keys=True) for name, c in cases.items()}
    ref = next(iter(blocks.values()), "")
    return [name for name, b in blocks.items() if b != ref]


def compare(case, base):
    a = {r["iter"]: r["loss"] for r in case["rows"]}
    b = {r["iter"]: r["loss"] for r in base["rows"]}
    common = sorted(set(a) & set(b))
    diffs = [(abs(a[i] - b[i]), i) for i in common]
    times = [r["step_time_s"] for r in case["rows"][1:] if r["step_time_s"] is not None]
    mems = [r["peak_memory_mb"] for r in case["rows"] if r["peak_memory_mb"] is not None]
    worst = max(diffs) if diffs else (float("nan"), -1)
    return {
        "steps": len(case["rows"]),
        "common_steps": len(common),
        "first_loss": case["rows"][0]["loss"] if case["rows"] else float("nan"),
        "final_loss": case["rows"][-1]["loss"] if case["rows"] else float("nan"),
        "max_abs_diff": worst[0],
        "max_abs_diff_step": worst[1],
        "mean_abs_diff": statistics.fmean(d for d, _ in diffs) if diffs else float("nan"),
        "final_delta": (a[common[-1]] - b[common[-1]]) if common else float("nan"),
        "median_step_time_s": statistics.median(times) if times else float("nan"),
        "peak_memory_mb": max(mems) if mems else float("nan"),
    }, [(i, a[i] - b[i]) for i in common]


def try_plots(out_dir: Path, cases, deltas, baseline):
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return False
    fig, ax = plt.subplots(figsize=(7, 4))
    for name, c in cases.items():
        ax.plot([r["iter"] for r in c["rows"]], [r["loss"] for r in c["rows"]], label=c["cfg"].get("case_label", name), lw=1)
    ax.set_xlabel("step"); ax.set_ylabel("loss"); ax.legend(fontsize=7); fig.tight_layout()
    fig.savefig(out_dir / "loss_curves.png", dpi=150); plt.close(fig)
    fig, ax = plt.subplots(figsize=(7, 4))
    for name, d in deltas.items():
        if name != baseline:
            ax.plot([i for i, _ in d], [v for _, v in d], label=name, lw=1)
    ax.axhline(0, color="k", lw=0.5); ax.set_xlabel("step"); ax.set_ylabel(f"loss - loss({baseline})"); ax.legend(fontsize=7)
    fig.tight_layout(); fig.savefig(out_dir / "loss_delta.png", dpi=150); plt.close(fig)
    return True


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--result_dir", default=str(HERE / "results"))
    ap.add_argument("--config_dir", default=str(HERE / "configs"))
    ap.add_argument("--output_dir", default=None)
    ap.add_argument("--baseline", default="seq_fsdp")
    ap.add_argument("--cases", nargs="*", default=None)
    ap.add_argument("--tolerance", type=float, default=None, help="fail when a case's max |loss difference| exceeds it")
    a = ap.parse_args(argv)
    result_dir, out_dir = Path(a.result_dir), Path(a.output_dir or a.result_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cases = load_cases(result_dir, Path(a.config_dir), set(a.cases) if a.cases else None)
    if a.baseline not in cases:
        print(f"baseline case {a.baseline!r} has no loss.csv under {result_dir}", file=sys.stderr)
        return 2
    mism = activation_mismatches(cases)
    summary, deltas = [], {}
    for name, c in cases.items():
        row, d = compare(c, cases[a.baseline])
        deltas[name] = d
        summary.append({"case": name, "label": c["cfg"].get("case_label", name), "topology": c["cfg"].get("topology_label", ""),
                        "finished": c["ok"], **row})
    with open(out_dir / "summary.csv", "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(summary[0].keys()))
        w.writeheader(); w.writerows(summary)
    plotted = try_plots(out_dir, cases, deltas, a.baseline)
    if not plotted:
        with open(out_dir / "loss_delta.csv", "w", newline="") as f:
            w = csv.writer(f); w.writerow(["case", "iter", "loss_minus_baseline"])
            for name, d in deltas.items():
                w.writerows([name, i, v] for i, v in d)
    failed = [r["case"] for r in summary if a.tolerance is not None and r["case"] != a.baseline and not (r["max_abs_diff"] <= a.tolerance)]
    lines = [f"# Loss consistency against `{a.baseline}`", "",
             "| case | topology | steps | final loss | max abs diff (step) | mean abs diff | final delta | median step s | peak MB |",
             "|---|---|---|---|---|---|---|---|---|"]
    for r in summary:
        lines.append(f"| {r['label']} | {r['topology']} | {r['steps']} | {r['final_loss']:.6g} | {r['max_abs_diff']:.3g} ({r['max_abs_diff_step']}) | "
                     f"{r['mean_abs_diff']:.3g} | {r['final_delta']:+.3g} | {r['median_step_time_s']:.4g} | {r['peak_memory_mb']:.6g} |")
    lines += ["", f"Activation settings identical across cases: {'yes' if not mism else 'NO (' + ', '.join(mism) + ')'}",
              f"Tolerance: {a.tolerance if a.tolerance is not None else 'none (informational)'}"
              + ("" if not failed else f"; exceeded by {', '.join(failed)}"),
              f"Plots: {'loss_curves.png, loss_delta.png' if plotted else 'matplotlib not available; see loss_delta.csv'}"]
    (out_dir / "report.md").write_text("\n".join(lines) + "\n")
    print("\n".join(lines))
    return 1 if (failed or mism) else 0


if __name__ == "__main__":
    sys.exit(main())
