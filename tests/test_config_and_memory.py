"""Pure-function units: padding, config validation, rank algebra, activation config, recompute scheduler, LR."""
import math

import pytest

from terra_b200.config import get_model_archi_params_and_other_params
from terra_b200.memory.activation import (activation_config_for_layer, activation_config_for_sampling,
                                          normalize_activation_config, normalize_activation_mode)
from terra_b200.memory.selective_recompute import SelectiveRecomputeScheduler
from terra_b200.optim.utils import get_finetune_lr_by_global_step, get_lr_by_global_step
from terra_b200.parallel.rank_manager import Topology
from terra_b200.utils.padding import compute_auto_padded_shape, get_padded_shape


def test_padding_rules():
    need, pad, shape = get_padded_shape(2041, 4320, 4, 8, padding_scale=2)
    assert shape == (2048, 4352) and need and pad == (16, 16, 3, 4)
    need, pad, shape = get_padded_shape(128, 256, 4, 8, padded_shape=(128, 256))
    assert not need and shape == (128, 256)
    with pytest.raises(ValueError):
        get_padded_shape(128, 256, 4, 8, padded_shape=(64, 256))
    assert compute_auto_padded_shape(2048, 4320, 4, 8, 2, (8, 1), (8, 1), "terra_m1_ragged_auto") == (2048, 4352)
    assert compute_auto_padded_shape(720, 1440, 4, (8, 12), 2, (8, 1), (8, 1), "terra_m1_ragged_auto") == (768, 1440)
    assert compute_auto_padded_shape(2041, 4320, 4, 32, 2, (8, 1), (8, 1), "terra_m1_ragged_auto") == (2048, 4352)


def test_padding_matches_reference_when_installed():
    from baseline import ref_import

    if not ref_import.available():
        pytest.skip("reference not installed")
    ref_import.enable()
    from models.model_utils.get_model import _compute_auto_padded_shape as ref_auto
    from utils import get_padded_shape as ref_pad

    for (h, w, p, ws, scale) in [(2041, 4320, 4, 8, 2), (721, 1440, 4, 8, 1), (100, 300, 2, 6, 2)]:
        assert get_padded_shape(h, w, p, ws, scale) == ref_pad(h, w, p, ws, scale)
    for mode, topo in [("terra_m1_ragged_auto", (8, 1)), ("terra_m1_regular", (4, 1)), ("regular", (2, 2)),
                       ("terra_m1_ragged_row", (6, 1)), ("ragged_round_robin", (8, 1))]:
        wp = (topo[0] * topo[1], 1)
        got = compute_auto_padded_shape(2041, 4320, 4, 8, 2, wp, topo, mode)
        assert got == ref_auto(2041, 4320, 4, 8, "credit_hierarchical_swin", wp, topo, mode), (mode, got)


BASE = dict(task_type="glorys", model_architecture="credit_hierarchical_swin", model_type="parallel", height=2048,
            width=4320, num_channels=186, patch_size=4, embedding_dim=384, depths=[2, 6, 6, 2], num_heads=[6, 12, 24, 12],
            num_layers=16, window_size=8, padding_policy="auto", window_assignment_mode="terra_m1_ragged_auto")


def test_config_resolution_high_res_2x2x2():
    cfg = dict(BASE, wp_topo="(8, 1)", xfmr_wp_topo="(2, 1)", xfmr_sp_size=2, tensor_parallel_size=2)
    archi, other = get_model_archi_params_and_other_params("glorys", cfg, 1, 8)
    assert archi["padded_shape"] == (2048, 4352) and archi["num_layers"] == 16
    assert other["wp_topo"] == (8, 1) and other["xfmr_wp_topo"] == (2, 1)
    assert archi["padding_spec"]["num_windows"] == (32, 68)
    with pytest.raises(ValueError):                    # product rule
        get_model_archi_params_and_other_params("glorys", dict(cfg, xfmr_sp_size=4), 1, 8)
    with pytest.raises(ValueError):                    # the all-to-all SP of the reference would need heads % 4 == 0
        get_model_archi_params_and_other_params("glorys", dict(cfg, strict_ulysses_heads=True), 1, 8)
    with pytest.raises(ValueError):
        get_model_archi_params_and_other_params("glorys", dict(cfg, window_topology="mn"), 1, 8)


def test_rank_algebra_roundtrip():
    for placement in ("tp_first", "sp_first"):
        t = Topology(dp_size=2, mp_size=1, wp_topo=(8, 1), xfmr_wp_topo=(2, 1), xfmr_sp_size=2, xfmr_tp_size=2,
                     sp_tp_placement=placement)
        seen = set()
        for wg in range(2):
            for sp in range(2):
                for tp in range(2):
                    r = t.xfmr_coord_to_wp_rank(wg, sp, tp)
                    assert t.wp_rank_to_xfmr_coord(r) == (wg, sp, tp)
                    seen.add(r)
        assert seen == set(range(8))
        assert t.global_rank(1, 0, 3) == 11 and t.split_rank(11) == (1, 0, 3)
        for groups in (t.dp_groups(), t.wp_groups(), t.sp_groups(), t.tp_groups(), t.tp_param_groups(),
                       t.full_param_replica_groups(), t.tp_param_replica_groups(), t.window_group_groups()):
            flat = sorted(r for g in groups for r in g)
            assert flat == sorted(list(range(16)) * (len(flat) // 16))
    assert Topology(wp_topo=(4, 1), xfmr_wp_topo=(2, 1), xfmr_tp_size=2).tp_groups() == [[0, 1], [2, 3]]
    with pytest.raises(ValueError):
        Topology(wp_topo=(4, 1), xfmr_wp_topo=(2, 1), xfmr_tp_size=4)


def test_activation_config_normalisation():
    assert normalize_activation_mode("torch") == "torch_recompute"
    assert normalize_activation_mode("cpu_offload_boundary") == "cpu_boundary_offload_recompute"
    with pytest.raises(ValueError):
        normalize_activation_mode("bogus")
    off = normalize_activation_config({"activation": {"mode": "none"}})
    assert not off["enabled"] and off["checkpoint_layers"] == []
    cfg = normalize_activation_config({"activation": {
        "mode": "torch_recompute", "policy": "larger_wrapper", "checkpoint_layers": ["D1", "0-3", 5, "U0"],
        "layer_modes": {"cpu_boundary_offload": [0], "5": "none"}, "sampling_modes": {"down": "boundary_offload"}}})
    assert cfg["checkpoint_segments"] == [(0, 4), (5, 6)]
    assert cfg["checkpoint_down_mode"] == "D1" and cfg["checkpoint_up_mode"] == "U0"
    assert activation_config_for_layer(cfg, 0)["mode"] == "cpu_boundary_offload_recompute"
    assert activation_config_for_layer(cfg, 5)["mode"] == "none"
    assert activation_config_for_sampling(cfg, "down")["mode"] == "cpu_boundary_offload_recompute"
    assert activation_config_for_sampling(cfg, "up")["mode"] == "torch_recompute"
    legacy = normalize_activation_config({"selective_recompute": {"enabled": True, "impl": "torch", "block_indices": [1, 2]}})
    assert legacy["mode"] == "torch_recompute" and legacy["checkpoint_layers"] == [1, 2]
    with pytest.raises(ValueError):
        normalize_activation_config({"activation": {"mode": "torch", "checkpoint_sampling_blocks": True}})


def test_recompute_scheduler_segments():
    s = SelectiveRecomputeScheduler({"mode": "torch", "policy": "uniform", "checkpoint_every_n_layers": 3}, depth=7)
    assert list(s.execution_segments()) == [(0, 1, True), (1, 2, False), (2, 3, False), (3, 4, True), (4, 5, False),
                                            (5, 6, False), (6, 7, True)]
    s = SelectiveRecomputeScheduler({"mode": "torch", "checkpoint_layers": ["1-2", 4]}, depth=6)
    assert list(s.execution_segments()) == [(0, 1, False), (1, 3, True), (3, 4, False), (4, 5, True), (5, 6, False)]
    s.set_checkpoint_plan(["0-1", "3-5"], activation_mode="cpu_boundary_offload_recompute",
                          segment_activation_modes=["torch", "boundary_offload"])
    assert s.checkpoint_segments == [(0, 2), (3, 6)]
    assert s.config_for_block(0)["mode"] == "torch_recompute"
    assert s.config_for_block(3)["mode"] == "cpu_boundary_offload_recompute"
    with pytest.raises(ValueError):
        SelectiveRecomputeScheduler({"mode": "torch", "checkpoint_layers": ["2-4", "3-5"]}, depth=8)
    assert list(SelectiveRecomputeScheduler(None, depth=2).execution_segments()) == [(0, 1, False), (1, 2, False)]
    full = SelectiveRecomputeScheduler({"mode": "torch"}, depth=3)
    assert full.checkpoint_segments == [(0, 1), (1, 2), (2, 3)]


def test_lr_schedules():
    assert get_lr_by_global_step("glorys", 0, 1e-3, 10, 2) == 0.0
    assert get_lr_by_global_step("glorys", 5, 1e-3, 10, 2) == pytest.approx(5e-4)
    assert get_lr_by_global_step("glorys", 10, 1e-3, 10, 2) == pytest.approx(1e-3)
    end = get_lr_by_global_step("glorys", 2 * 594, 1e-3, 10, 2)
    assert end == pytest.approx(1e-6)
    mid = get_lr_by_global_step("glorys", 10 + (2 * 594 - 10) // 2, 1e-3, 10, 2)
    assert mid == pytest.approx(1e-6 + (1e-3 - 1e-6) * 0.5, rel=1e-6)
    assert get_finetune_lr_by_global_step(3, 1e-3, 6) == pytest.approx(5e-4)
    assert get_finetune_lr_by_global_step(60, 1e-3, 6) == 1e-3


def test_bind_to_gpu_numa_with_fake_nvml(monkeypatch):
    """CPU affinity follows the mask a (fake) NVML reports for the GPU; GPU settings are never written."""
    import os
    import sys
    import types

    from terra_b200 import distributed as D

    if not hasattr(os, "sched_setaffinity"):
        return
    allowed = sorted(os.sched_getaffinity(0))
    want = set(allowed[: max(1, len(allowed) // 2)])
    calls = []
    fake = types.SimpleNamespace(
        nvmlInit=lambda: calls.append("init"), nvmlShutdown=lambda: calls.append("shutdown"),
        nvmlDeviceGetHandleByIndex=lambda i: ("h", i),
        nvmlDeviceGetCpuAffinity=lambda h, n: [sum(1 << (c - 64 * w) for c in want if 64 * w <= c < 64 * (w + 1)) for w in range(n)])
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,5")
    assert D._physical_gpu_index(1) == 5
    before = os.sched_getaffinity(0)
    try:
        assert D.bind_to_gpu_numa(0) is True
        assert os.sched_getaffinity(0) == want
        assert calls == ["init", "shutdown"]
        monkeypatch.setenv("TERRA_NUMA_BIND", "0")
        assert D.bind_to_gpu_numa(0) is False
    finally:
        os.sched_setaffinity(0, before)


def test_large_window_attention_core_matches_reference():
    """Windows above the kernel's 128 tokens run on the fused-attention core; same result as the explicit softmax."""
    import torch

    from terra_b200.ops.attention import (WindowGeometry, attention_core_sdpa, window_attention_reference)

    torch.manual_seed(0)
    geo = WindowGeometry(1, 2, 2, 12, 12)                      # 144 tokens per window
    C, heads = 32, 4
    qkv = torch.randn(1, 4, geo.N, 3 * C)
    table = torch.randn((2 * 12 - 1) ** 2, heads) * 0.2
    for shifted in (False, True):
        ref = window_attention_reference(qkv, geo, heads, shifted, table, True, 8 ** -0.5)
        got = window_attention_reference(qkv, geo, heads, shifted, table, True, 8 ** -0.5, core=attention_core_sdpa)
        assert torch.allclose(ref, got, atol=1e-5, rtol=1e-4)


def test_show_gradient_lists_first_and_last_block():
    import torch

    from terra_b200.runtime.grad_debug import install_grad_hooks, show_gradient

    class Blk(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1 = torch.nn.LayerNorm(4)
            self.norm2 = torch.nn.LayerNorm(4)

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.patch_embed = torch.nn.Linear(4, 4)
            self.blocks = torch.nn.ModuleList([Blk() for _ in range(3)])

        def forward(self, x):
            x = self.patch_embed(x)
            for b in self.blocks:
                x = b.norm2(b.norm1(x))
            return x

    m = M()
    seen = []
    handles = install_grad_hooks(m, limit=3, printer=seen.append)
    m(torch.randn(2, 4)).sum().backward()
    assert len(seen) == 3 and all(s.startswith("[grad hook]") for s in seen)
    for h in handles:
        h.remove()
    lines = show_gradient(m, printer=lambda s: None)
    names = [ln.split()[3].rstrip(":") for ln in lines]
    assert "patch_embed.weight" in names and "blocks.0.norm1.weight" in names and "blocks.2.norm2.bias" in names
    assert not any(n.startswith("blocks.1.") for n in names)


def test_exposed_comm_accounting():
    from terra_b200.profiler.exposed_comm import account, is_comm_kernel, union_length

    assert union_length([(0, 2), (1, 3), (5, 6)]) == 4
    assert is_comm_kernel("ncclDevKernel_AllReduce_Sum_f32_RING_LL") and is_comm_kernel("tb::peer_barrier_kernel")
    assert is_comm_kernel("tb::(anonymous namespace)::halo_push_kernel(tb::HaloPushArgs)")
    assert is_comm_kernel("tb::(anonymous namespace)::peer_allreduce_small_kernel") and is_comm_kernel("peer_gather_indexed_kernel")
    assert not is_comm_kernel("void tb::gemm_tcgen05_kernel<192, 1, false>") and not is_comm_kernel("dist_adamw_kernel")
    r = account([("gemm", 0.0, 4.0), ("ncclDevKernel_SendRecv", 3.0, 6.0), ("layernorm", 7.0, 8.0),
                 ("tb::peer_barrier_kernel", 8.0, 9.0)])
    assert r["span"] == 9.0 and r["compute_busy"] == 5.0 and r["comm_busy"] == 4.0
    assert r["comm_hidden"] == 1.0 and r["exposed"] == 4.0


def test_every_shipped_config_parses():
    """All YAML files under configs/ resolve to model / layout parameters for the world size their layout names."""
    import glob
    import os
    import re

    import yaml

    from terra_b200.config import get_model_archi_params_and_other_params

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "configs", "**", "*.yaml"), recursive=True))
    assert len(files) >= 9
    for f in files:
        cfg = yaml.safe_load(open(f))
        world = 1
        if cfg.get("model_type") == "parallel":
            a, b = (int(v) for v in re.findall(r"\d+", str(cfg.get("wp_topo", "(1, 1)")))[:2])
            world = a * b
        archi, other = get_model_archi_params_and_other_params(cfg.get("task_type", "glorys"), cfg, 1, world)
        ph, pw = archi["padded_shape"]
        unit = archi["patch_size"] * 2 * (archi["window_size"] if isinstance(archi["window_size"], int) else archi["window_size"][0])
        assert ph > 0 and pw > 0 and ph % unit == 0, (f, archi["padded_shape"], unit)


def test_bench_clock_sampler_parses_nvidia_smi_rows(tmp_path):
    """The clocks record of the benchmark line: median SM clock, maximum clock, throttle reasons seen."""
    import sys

    root = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    sys.path.insert(0, root)
    import bench

    class Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    f = tmp_path / "clocks.csv"
    f.write_text("0, 1965, 1965, 612.3, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                 "0, 1905, 1965, 998.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                 "0, 1950, 1965, 700.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n"
                 "garbage line\n")
    s = bench.ClockSampler(0)
    s.proc, s.path = Done(), str(f)
    out = s.stop()
    assert out["sm_mhz"] == 1950.0 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"] and out["samples"] == 3
    cfg = bench.flagship_config(8)
    assert cfg["wp_topo"] == "(8, 1)" and cfg["optimizer_config"] == 6 and cfg["height"] == 2048 and cfg["num_channels"] == 186


def test_nvtx_decorator_is_a_no_op_by_default():
    from terra_b200.utils import nvtx

    def f(x):
        return x + 1

    assert nvtx.ENABLED is False and nvtx.nvtx_range("t")(f) is f


def test_lead_schedules_parse_the_reference_formats_and_drive_the_model():
    """Per-lead activation plans: dict and list forms, ranges, aliases, string layer lists, validation; applied to a
    model only when the plan changes; sampling modes return to the base configuration outside their range."""
    import pytest
    from terra_b200.memory.lead_schedule import LeadScheduler, parse_lead_checkpoint_schedule, parse_lead_sampling_schedule
    from terra_b200.models import SequentialHierarchicalSwin

    act = {"mode": "torch_recompute", "offload": {"min_numel": 7},
           "lead_checkpoint_schedule": [
               {"lead": 3, "end": 4, "layers": "0-1, 3", "mode": "cpu_boundary_offload_recompute", "label": "late"},
               {"start": 2, "checkpoint_layers": [0], "segment_activation_modes": "torch_recompute"}],
           "lead_sampling_checkpoint_schedule": {"3-4": {"down": "d1", "up": "U0"}}}
    plans = parse_lead_checkpoint_schedule(act)
    assert [(p.lead_start, p.lead_end, p.label) for p in plans] == [(2, 2, "lead2-2"), (3, 4, "late")]
    assert plans[1].checkpoint_layers == ["0-1", "3"] and plans[1].offload == {"min_numel": 7}
    assert plans[1].segment_activation_modes == ["cpu_boundary_offload_recompute"] * 2
    assert parse_lead_checkpoint_schedule({"lead_checkpoint_layers": {"1-2": [0, 1]}})[0].lead_end == 2      # older key
    smp = parse_lead_sampling_schedule(act)
    assert (smp[0].down, smp[0].up, smp[0].lead_start, smp[0].lead_end) == ("D1", "U0", 3, 4)
    with pytest.raises(ValueError, match="must match checkpoint_layers"):
        parse_lead_checkpoint_schedule({"lead_checkpoint_schedule": [{"lead": 1, "layers": [0, 1], "segment_activation_modes": ["none"]}]})
    with pytest.raises(ValueError, match="missing checkpoint_layers"):
        parse_lead_checkpoint_schedule({"lead_checkpoint_schedule": [{"lead": 1}]})
    with pytest.raises(ValueError, match="must contain down or up"):
        parse_lead_sampling_schedule({"lead_sampling_checkpoint_schedule": {"1": {"offload": {}}}})
    with pytest.raises(ValueError, match="unsupported axes"):
        parse_lead_sampling_schedule({"lead_sampling_checkpoint_schedule": [{"lead": 1, "down": "D0", "sampling_modes": {"side": "x"}}]})

    model = SequentialHierarchicalSwin(padding_scale=1, num_channels=8, patch_size=4, window_size=8, height=64, width=128,
                                       embedding_dim=32, num_heads=2, num_layers=4,
                                       recompute_config={"mode": "torch_recompute", "checkpoint_layers": []})
    sched = LeadScheduler(model, act)
    rs = model.recompute_scheduler
    sched.before_lead(0)                                   # lead 1: nothing scheduled, the installed plan stays
    assert rs.checkpoint_segments == [] and model.checkpoint_down_mode == "none"
    sched.before_lead(1)                                   # lead 2
    assert rs.checkpoint_segments == [(0, 1)] and sched.describe(1)["checkpoint_label"] == "lead2-2"
    sched.before_lead(2)                                   # lead 3: offload plan + sampling checkpoints
    assert rs.checkpoint_segments == [(0, 2), (3, 4)] and rs.mode == "cpu_boundary_offload_recompute"
    assert (model.checkpoint_down_mode, model.checkpoint_up_mode) == ("D1", "U0")
    row = sched.describe(2)
    assert row["lead"] == 3 and row["sampling_down"] == "D1" and row["checkpoint_layers"] == '["0-1", "3"]'
    sched.before_lead(4)                                   # lead 5: sampling back to the base, transformer plan kept
    assert (model.checkpoint_down_mode, model.checkpoint_up_mode) == ("none", "none")
    assert rs.checkpoint_segments == [(0, 2), (3, 4)] and sched.describe(4)["checkpoint_label"] == "late"
