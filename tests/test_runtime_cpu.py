"""Step-runtime helpers that need no GPU."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_arena_gradient_report_lists_every_parameter_up_to_the_limit():
    """``DEBUG_GRAD_HOOK`` where no autograd hook can fire (gradients written in place by kernels): the sums are read
    from the parameters' gradient views after the backward pass, with the run-wide line limit."""
    from terra_b200.runtime import grad_debug

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2))
    net(torch.randn(5, 4)).sum().backward()
    grad_debug._arena_lines["n"] = 0
    seen = []
    lines = grad_debug.report_arena_gradients(net, limit=3, printer=seen.append)
    assert len(lines) == 3 == len(seen) and lines[0].startswith("[grad hook] 0.weight: ")
    want = net[0].weight.grad.double().sum().item()
    assert abs(float(lines[0].split(": ")[1]) - want) <= 1e-7 * max(1.0, abs(want))      # the line prints 9 digits
    assert grad_debug.report_arena_gradients(net, limit=3, printer=seen.append) == []      # the limit holds over the run
    grad_debug._arena_lines["n"] = 0


def test_memory_timeline_intervals_outputs_and_filters(tmp_path, monkeypatch):
    """The timeline on a machine without a GPU records the event stream with zero sizes; with a stand-in for the
    allocator readings it must attribute interval peaks to the closing event, keep the peaks its resets fold away,
    merge the semantic context into events, and write CSV / summary / event table with hidden classes filtered."""
    from terra_b200.profiler import memory_timeline as M

    tl = M.CudaMemoryTimeline(None, enabled=True, output_dir=str(tmp_path), tag="t")
    assert tl.force_cpu or tl.enabled
    levels = iter([(10, 20, 10), (12, 20, 12), (30, 40, 55), (14, 40, 60), (14, 40, 14), (9, 40, 14), (9, 40, 14)])

    def fake_snapshot():
        a, r, p = next(levels)
        return float(a), float(r), float(p), float(r) + 5.0, 5.0

    monkeypatch.setattr(tl, "_snapshot", fake_snapshot)
    M.set_memory_timeline_context(lead_idx=3, execution_phase="forward")
    with tl.iteration(M.MEMORY_TIMELINE_OUTPUT_START_ITER):
        occ = M.new_memory_timeline_occurrence("block0")
        M.mark_memory_timeline("primitive_forward_pre", "block0", occurrence_id=occ, primitive_kind="transformer")
        M.mark_memory_timeline("module_fwd_pre", "attn")                      # hidden class by default
        M.mark_memory_timeline("primitive_forward_post", "block0", occurrence_id=occ, primitive_kind="transformer")
        M.mark_memory_timeline("after_forward")
        M.set_memory_timeline_context(execution_phase=None)
        M.mark_memory_timeline("before_backward")
    M.set_memory_timeline_context(lead_idx=None)
    phases = [e["phase"] for e in tl.events]
    assert phases == ["iter_start", "primitive_forward_pre", "module_fwd_pre", "primitive_forward_post", "after_forward",
                      "before_backward", "iter_end"]
    closer = tl.events[3]["meta"]
    assert closer["interval_kind"] == "primitive_forward" and closer["interval_start_allocated_mib"] == 12.0
    assert closer["interval_peak_allocated_mib"] == 60.0 and closer["interval_peak_rise_mib"] == 48.0
    assert closer["lead_idx"] == 3 and closer["execution_phase"] == "forward"
    assert "execution_phase" not in tl.events[5]["meta"]                      # removed from the context
    assert tl.overall_peak_allocated_mib == 60.0 == tl.iteration_peak_allocated_mib
    rows = tl.primitive_intervals()
    assert len(rows) == 1 and rows[0]["interval_peak_mib"] == 60.0 and rows[0]["direction"] == "forward"
    assert [e["phase"] for e in tl.visible_events()] == [p for p in phases if p != "module_fwd_pre"]
    made = tl.write_outputs()
    assert {"csv", "summary", "primitive_summary", "event_table"} <= set(made)
    table = open(made["event_table"]).read()
    assert "primitive_forward_post" in table and "module_fwd_pre" not in table and "rise +48.0" in table
    assert "module_fwd_pre" in open(made["csv"]).read()                       # the CSV keeps every event
    assert "overall_peak_allocated_mib: 60.0" in open(made["summary"]).read()
    assert M.event_class("sampling_down_enter") == "sampling_boundary" and M.event_class("sampling_conv1") == "sampling_internal"
    assert not M.memory_timeline_iteration_enabled(M.MEMORY_TIMELINE_OUTPUT_START_ITER + M.MEMORY_TIMELINE_OUTPUT_MAX_ITERS)


def test_balanced_split_fills_whole_rounds_of_the_persistent_grid():
    """Split-K policy of the convolution weight gradient: ``tiles * split`` work items over 148 persistent CTAs."""
    from terra_b200.ops.conv import balanced_split

    def rounds_per_unit_work(tiles, s):
        return -(-tiles * s // 148) / s

    # 54 tiles (9 taps x 3 x 2 at 384 channels): a split of 2 would run two rounds, the second nearly empty
    s = balanced_split(54, 8704)
    assert s == 8 and rounds_per_unit_work(54, s) < 0.38 < rounds_per_unit_work(54, 2)
    assert balanced_split(81, 8704) == 9
    assert balanced_split(148, 8704) == 1              # one full round already
    assert balanced_split(54, 3) <= 3                   # never more splits than k-blocks
    for tiles in (6, 18, 24, 48, 72, 81, 148, 149, 300):
        s = balanced_split(tiles, 100000)
        ideal = tiles / 148
        assert rounds_per_unit_work(tiles, s) <= 1.15 * max(ideal, 1 / 64) + 1e-9, (tiles, s)


def test_trainer_checkpoint_round_trip_through_the_public_api(tmp_path):
    """``Trainer.save_checkpoint`` / ``load_checkpoint``: weights and optimizer state come back, and the next step
    after a resume equals the next step of the uninterrupted run."""
    from terra_b200.api import Trainer

    cfg = dict(task_type="glorys", model_architecture="credit_hierarchical_swin", model_type="sequential", height=64,
               width=128, num_channels=8, patch_size=4, embedding_dim=32, num_layers=2, num_heads=2, window_size=8,
               padding_policy="auto", optimizer_config=4, precision="fp32", loss_func="MSE", learning_rate=1e-3,
               train_path=str(tmp_path), description="api_ckpt")
    t = Trainer(cfg)
    batches = [t.synthetic_batch(sample=i, pin=False) for i in range(3)]
    t.step(batches[0])
    t.step(batches[1])
    path = t.save_checkpoint(epoch=0, loss=1.0)
    assert path is not None and path.endswith("epoch0.pth")
    want = t.step(batches[2])
    t2 = Trainer(dict(cfg), seed=999)                    # different initial weights: everything must come from the file
    epoch, gstep, loss = t2.load_checkpoint(epoch=0)
    assert (epoch, gstep, loss) == (0, 2, 1.0)
    got = t2.step(batches[2])
    assert abs(got - want) <= 1e-6 * max(1.0, abs(want)), (got, want)


def test_small_utilities():
    from terra_b200.utils.misc import check_parallel_config, get_task_partition, sort_key

    spans = [get_task_partition(r, 8, 331) for r in range(8)]
    assert spans[0] == (0, 41) and spans[-1] == (289, 331)
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))                  # contiguous, nothing lost
    assert [e - s for s, e in spans] == [41] * 5 + [42] * 3
    assert get_task_partition(3, 4, 331, div_10=True) == (25, 34)
    assert sorted(["/d/10.nc", "/d/9.nc", "/d/100.nc"], key=sort_key) == ["/d/9.nc", "/d/10.nc", "/d/100.nc"]
    check_parallel_config(2, 1, (4, 1), (1, 1), 8, 2048, 4320, 4, 8, padding_scale=2)
    import pytest

    with pytest.raises(ValueError, match="world_size"):
        check_parallel_config(2, 1, (4, 1), (1, 1), 16, 2048, 4320, 4, 8)
    with pytest.raises(ValueError, match="window grid"):
        check_parallel_config(1, 1, (7, 1), (1, 1), 7, 2048, 4320, 4, 8, padding_scale=2)


def test_buffer_helpers():
    from terra_b200.utils import buffers as Bf

    a = Bf.get_preallocated_buffer((2, 3), torch.float32, "cpu", key="x")
    assert Bf.get_preallocated_buffer((2, 3), torch.float32, "cpu", key="x") is a
    assert Bf.get_preallocated_buffer((2, 3), torch.float32, "cpu", key="y") is not a
    assert Bf.get_preallocated_buffer((2, 4), torch.float32, "cpu", key="x").shape == (2, 4)
    t = torch.zeros(4, 6).t()                                   # non-contiguous: strides are kept
    h = Bf.new_cpu_buffer_like(t)
    assert h.shape == t.shape and h.stride() == t.stride() and h.device.type == "cpu"
    assert Bf.get_cuda_stream("cpu") is None or torch.cuda.is_available()
    Bf.release_preallocated_buffers()


def test_harness_metric_files_use_the_reference_columns(tmp_path):
    """The harnesses' CSV columns and JSON keys, in the reference's names and order (train_scripts/test_pretrain.py:555-660,
    train_scripts/test_finetune.py:1105-1206 there), with this framework's additional columns after them."""
    import argparse
    import csv
    import json
    import types

    import torch

    sys.path.insert(0, ROOT)
    from train_scripts import metrics as M
    from terra_b200.profiler.flops_profiler import FlopsSummary

    archi = dict(height=100, width=200, padded_shape=[128, 256], initial_padding=[14, 14, 28, 28], padding_policy="auto",
                 padding_spec=dict(need_padding=True, patch_token_resolution=(32, 64), transformer_token_resolution=(16, 32),
                                   num_windows=(2, 4), transformer_downsample_scale=2))
    pad = M.padding_facts(archi)
    assert pad["padded_shape"] == (128, 256) and pad["input_shape"] == (100, 200) and pad["need_padding"] is True
    assert abs(pad["padding_overhead_pct"] - (128 * 256 / 20000 - 1) * 100) < 1e-9

    r = M.finetune_row(0, 4, "mean", 0.5, 3.0, torch.bfloat16, 10.0, 2.0, 1.5, 0.1, local_flops_per_step=4e12, h2d_bytes=7)
    assert list(r)[:len(M.FINETUNE_COLUMNS)] == list(M.FINETUNE_COLUMNS) and r["h2d_bytes"] == 7
    assert r["loss_per_lead"] == 0.5 and r["loss_sum_estimated"] == 2.0 and r["rest_time_s"] == 0.5 and r["flops_tflops"] == 2.0
    r = M.finetune_row(0, 4, "sum", 2.0, 3.0, torch.float32, 10.0, 2.0, None, None)
    assert r["loss_per_lead"] == 0.5 and r["loss_sum_estimated"] == 2.0 and r["rest_time_s"] is None and r["flops_tflops"] == 0.0

    ns = argparse.Namespace(metrics_csv=str(tmp_path / "a" / "m.csv"), metrics_json=None, metrics_no_json=False,
                            model_cfg="x.yaml", memory_timeline_csv=None)
    assert M.json_path_for(ns) == str(tmp_path / "a" / "m.json")
    assert M.json_path_for(argparse.Namespace(metrics_csv="m.csv", metrics_json="j.json", metrics_no_json=True)) is None

    model = torch.nn.Linear(3, 2)
    session = types.SimpleNamespace(
        model=model, archi=archi, world=1, dp=1, task_type="glorys", model_type="sequential",
        other=dict(wp_topo=[1, 1], xfmr_wp_topo=[1, 1], tensor_parallel_size=1),
        cfg=dict(optimizer_config=7, precision="bf16", micro_batch_size=1, padding_scale=1, num_layers=4))
    rows = [dict(iter=i, loss=1.0 - 0.1 * i, output_sum=2.0, output_dtype="torch.float32", peak_memory_mb=5.0,
                 step_time_s=0.25, forward_time_s=0.1) for i in range(2)]
    facts = M.gather_run_facts(session, rows, dict(offloaded_tensors=0))
    assert facts["parameter_count"]["global_parameter_count"] == 8 and facts["parameter_count"]["fsdp_group_size"] == 1
    assert facts["step_time_last_by_rank"] == [0.25] and facts["boundary_offload_stats_by_rank"] == [dict(offloaded_tensors=0)]
    M.write_pretrain_metrics(session, ns, rows, facts, FlopsSummary(enabled=False), extra=dict(final_loss=0.9))
    got = list(csv.DictReader(open(ns.metrics_csv)))
    assert list(got[0])[:len(M.PRETRAIN_COLUMNS)] == list(M.PRETRAIN_COLUMNS) and list(got[0])[-1] == "forward_time_s"
    assert got[1]["padded_shape"] == "(128, 256)" and got[1]["num_windows"] == "(2, 4)" and got[1]["iter"] == "1"
    meta = json.load(open(tmp_path / "a" / "m.json"))
    for k in ("model_cfg", "steps", "ranks_per_dp", "wp_topo", "padding_overhead_pct", "parameter_count",
              "parameter_count_method", "pre_wrap_parameter_counts_by_rank", "flops_profiler_enabled",
              "flops_profiler_world_avg_flops_per_step", "final_loss"):
        assert k in meta, k
    assert meta["steps"] == 2 and meta["padded_shape"] == [128, 256] and meta["flops_profiler_enabled"] is False

    ns.memory_timeline_csv = str(tmp_path / "a" / "leads.csv")
    lead_rows = [dict(iter=0, lead=1, checkpoint_label="lead1-1", loss=0.3, peak_memory_mb=1.0)]
    M.write_finetune_metrics(session, ns, [M.finetune_row(0, 2, "mean", 0.5, 3.0, "torch.float32", 10.0, 2.0, 1.0, 0.1)],
                             lead_rows, facts, FlopsSummary(enabled=False), 2, "mean", dict(input_double_buffer=True))
    assert list(csv.DictReader(open(ns.memory_timeline_csv)))[0]["checkpoint_label"] == "lead1-1"
    assert tuple(csv.DictReader(open(ns.memory_timeline_csv)).fieldnames) == M.LEAD_COLUMNS
    meta = json.load(open(tmp_path / "a" / "m.json"))
    assert meta["script"] == "test_finetune.py" and meta["lead_time"] == 2 and meta["input_double_buffer"] is True
    assert meta["parameter_count_by_rank"] == [8] and meta["test_iter_num"] == 1


def test_symmetric_memory_group_names_are_not_inherited_across_topologies():
    """torch's symmetric-memory layer registers a group under its NAME once and for all, and ``destroy_process_group``
    restarts the name counter: a group of a second topology in the same process would inherit the store, rank and size of
    a dead group of the first (its rendezvous then waits for ever). ``_register_group`` drops a name that is known for
    another group object before registering; the same object is registered once."""
    import types

    from terra_b200.parallel import nvlink

    calls = []
    fake = types.SimpleNamespace(_group_name_to_store={}, enable_symm_mem_for_group=None)

    def enable(name):
        calls.append(name)
        fake._group_name_to_store.setdefault(name, object())

    fake.enable_symm_mem_for_group = enable
    nvlink._GROUP_OF_NAME.clear()
    first = types.SimpleNamespace(group_name="1")
    nvlink._register_group(fake, first)
    store_a = fake._group_name_to_store["1"]
    nvlink._register_group(fake, first)                       # a second arena on the same group: nothing is dropped
    assert fake._group_name_to_store["1"] is store_a
    second = types.SimpleNamespace(group_name="1")            # another topology, the counter started again
    nvlink._register_group(fake, second)
    assert fake._group_name_to_store["1"] is not store_a and calls == ["1", "1", "1"]
    nvlink._GROUP_OF_NAME.clear()
