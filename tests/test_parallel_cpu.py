"""Multi-rank layouts on gloo CPU ranks against the single-rank model (same seeded weights, same data):
loss, output and the reduced gradients must agree."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys, json
    sys.path.insert(0, %(root)r)
    import torch, torch.distributed as dist
    from terra_b200.api import Trainer
    from terra_b200.data.synthetic import synthetic_batch, land_mask_for_rank, patchify_hwc
    from terra_b200.models import SequentialHierarchicalSwin
    from terra_b200.ops.loss import masked_loss

    cfg = dict(%(cfg)s)
    t = Trainer(cfg, data_parallel_group_size=1, backend="gloo")
    a = t.archi
    batch = t.synthetic_batch(0)
    # one forward/backward through the runtime pieces (no optimizer step, to compare raw gradients)
    from terra_b200.runtime.run_one_step import loss_scale_factor, grad_post_process, backbone_run, cal_loss
    t.optimizer.zero_grad()
    outs = backbone_run("glorys", t.model, batch, t.task_data)
    post = loss_scale_factor("parallel", "window_linear", t.manager, t.task_data, False)
    loss = cal_loss("glorys", outs, batch, t.task_data, torch.nn.MSELoss()) * post
    loss.backward()
    grad_post_process("parallel", (True, False, -1, False), t.model, t.manager, dp_average=True)
    rep = loss.detach().clone(); dist.all_reduce(rep)

    # single-rank oracle on the whole padded field, same seeded init
    H, W, C, p = a["height"], a["width"], a["num_channels"], a["patch_size"]
    ser = SequentialHierarchicalSwin(padding_scale=1, num_channels=C, patch_size=p, window_size=a["window_size"], height=H,
                                     width=W, embedding_dim=a["embedding_dim"], num_heads=a["num_heads"],
                                     num_layers=a["num_layers"], depths=a.get("depths"),
                                     padding_spec={"padded_shape": a["padded_shape"]})
    full = synthetic_batch(H, W, C, p, a["padded_shape"], a["initial_padding"], "sequential", 1, 0, 1, 0)
    mask, _ = land_mask_for_rank(H, W, C, p, a["padded_shape"], a["initial_padding"], "sequential")
    y = ser(full["input_tensor"]) * mask
    ref_loss = torch.nn.functional.mse_loss(y, full["label_tensor"])
    ref_loss.backward()

    # compare: loss, my stripe of the output, gradients of replicated parameters
    wp, r = t.manager.wp_size, t.manager.wp_rank
    rows = a["padded_shape"][0] // wp
    left, right, top, bottom = a["initial_padding"]
    ypad = torch.nn.functional.pad(y.detach(), (0, 0, left, right, top, bottom))
    mine_ref = patchify_hwc(ypad[:, r * rows:(r + 1) * rows], p)
    out_err = (outs[0].detach() - mine_ref).abs().max().item()
    sp = dict(ser.named_parameters())
    worst = 0.0
    names = {"patch_embed.weight": "patch_embed.linear.weight", "patch_recovery.weight": "patch_recovery.linear.weight",
             "patch_embed.bias": "patch_embed.linear.bias", "patch_recovery.bias": "patch_recovery.linear.bias"}
    checked = 0
    for n, q in t.model.named_parameters():
        if getattr(q, "terra_grad_reduce_group", None):
            continue      # TP shards are compared separately
        sn = names.get(n, n.replace(".conv.conv.", ".conv.").replace(".conv.weight", ".weight").replace(".conv.bias", ".bias") if ".b." in n else names.get(n, n.replace("down_blk.conv.conv", "down_blk.conv").replace("up_blk.conv.conv", "up_blk.conv")))
        if sn not in sp:
            continue
        g_ref = sp[sn].grad
        if g_ref is None or g_ref.abs().max() < 1e-9:
            continue
        worst = max(worst, ((q.grad - g_ref).abs().max() / (g_ref.abs().max() + 1e-12)).item())
        checked += 1
    print("RESULT " + json.dumps(dict(rank=dist.get_rank(), loss=rep.item(), ref_loss=ref_loss.item(), out_err=out_err,
                                      worst_grad_rel=worst, checked=checked,
                                      comms=sorted(c.__name__ for c, _ in getattr(t.model.pctx, "_comm_cache", {})))),
          flush=True)
    dist.destroy_process_group()
''')

BASE = ("task_type='glorys', model_architecture='credit_hierarchical_swin', model_type='parallel', height=128, width=256, "
        "num_channels=16, patch_size=4, embedding_dim=64, num_layers=2, num_heads=4, window_size=8, padding_policy='auto', "
        "optimizer_config=4, precision='fp32', loss_func='MSE', learning_rate=1e-4, land_mask='blobs', ")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _run(world, extra, code=None, **env_extra):
    code = code if code is not None else WORKER % dict(root=ROOT, cfg=BASE + extra)
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES="", **env_extra)
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                      text=True))
    results = []
    for p in procs:
        try:
            out, err = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        assert p.returncode == 0, err[-3000:]
        line = [ln for ln in out.splitlines() if ln.startswith("RESULT ")][-1]
        results.append(__import__("json").loads(line[len("RESULT "):]))
    return results


@pytest.mark.parametrize("world,extra", [
    (2, "wp_topo='(2, 1)', xfmr_wp_topo='(2, 1)', window_assignment_mode='terra_m1_ragged_auto'"),
    (2, "wp_topo='(2, 1)', xfmr_wp_topo='(2, 1)', window_assignment_mode='regular'"),
    (2, "wp_topo='(2, 1)', xfmr_wp_topo='(1, 1)', xfmr_sp_size=2, window_assignment_mode='terra_m1_ragged_auto'"),
    (2, "wp_topo='(2, 1)', xfmr_wp_topo='(1, 1)', tensor_parallel_size=2, window_assignment_mode='terra_m1_ragged_auto'"),
    (4, "wp_topo='(4, 1)', xfmr_wp_topo='(1, 1)', xfmr_sp_size=2, tensor_parallel_size=2, window_assignment_mode='terra_m1_ragged_auto'"),
])
def test_parallel_layout_matches_serial(world, extra):
    for res in _run(world, extra):
        assert abs(res["loss"] - res["ref_loss"]) < 1e-4 * max(1.0, abs(res["ref_loss"])), res
        assert res["out_err"] < 2e-3, res
        assert res["checked"] > 10 and res["worst_grad_rel"] < 2e-3, res
        # window groups without token shards exchange only the pieces of their shifted windows
        assert res["comms"] == (["_ShiftExchangeAttnComm"] if ("xfmr_wp_topo='(1, 1)'" not in extra and "sp_size" not in extra) else []), res


@pytest.mark.parametrize("world,extra,baseline", [
    (2, "wp_topo='(2, 1)', xfmr_wp_topo='(1, 2)', window_assignment_mode='regular'", "exchange"),          # column split
    (2, "wp_topo='(2, 1)', xfmr_wp_topo='(2, 1)', window_assignment_mode='ragged_round_robin'", "exchange"),
    (4, "wp_topo='(4, 1)', xfmr_wp_topo='(2, 2)', window_assignment_mode='regular'", "exchange"),          # 2-D blocks
    (3, "wp_topo='(3, 1)', xfmr_wp_topo='(3, 1)', window_assignment_mode='ragged_round_robin'", "exchange"),
    (2, "wp_topo='(2, 1)', xfmr_wp_topo='(1, 2)', window_assignment_mode='regular'", "gather"),            # the old baseline
    # with token shards: q rows of the own query slots and k / v rows of whole windows travel along their own routes
    (4, "wp_topo='(4, 1)', xfmr_wp_topo='(2, 1)', xfmr_sp_size=2, window_assignment_mode='terra_m1_ragged_auto'", "exchange-sp"),
    (4, "wp_topo='(4, 1)', xfmr_wp_topo='(1, 2)', xfmr_sp_size=2, window_assignment_mode='regular'", "exchange-sp"),
])
def test_non_contiguous_window_ownership_matches_serial(world, extra, baseline):
    """Ownership maps in which a rank's windows are not one range of the row-major order (column blocks, 2-D blocks,
    round robin): the shifted windows are put together from routed pieces (reference: core/window_parallel.py:26-266);
    ``TERRA_WP_BASELINE=gather`` keeps the gather-everything form."""
    want = {"exchange": ["_ShiftExchangeAttnComm"], "exchange-sp": ["_ShardedShiftExchangeAttnComm"], "gather": []}[baseline]
    for res in _run(world, extra, TERRA_WP_BASELINE=baseline.split("-")[0]):
        assert abs(res["loss"] - res["ref_loss"]) < 1e-4 * max(1.0, abs(res["ref_loss"])), res
        assert res["out_err"] < 2e-3 and res["checked"] > 10 and res["worst_grad_rel"] < 2e-3, res
        assert res["comms"] == want, res


def test_ragged_ownership_with_rectangular_windows_matches_serial():
    """The structure of the medium-resolution benchmark layout in small: 8 x 12 windows, a window grid (3 x 2) whose rows
    do not divide over the ranks, row-major ragged ownership (3 windows each: the ranks share a window row), hence the
    general stripe <-> window relayout and a halo that is part of a window row."""
    base = BASE.replace("height=128, width=256", "height=192, width=192").replace("window_size=8", "window_size=[8, 12]")
    assert base != BASE
    extra = "wp_topo='(2, 1)', xfmr_wp_topo='(2, 1)', window_assignment_mode='terra_m1_ragged_auto'"
    for res in _run(2, "", code=WORKER % dict(root=ROOT, cfg=base + extra)):
        assert abs(res["loss"] - res["ref_loss"]) < 1e-4 * max(1.0, abs(res["ref_loss"])), res
        assert res["out_err"] < 2e-3 and res["checked"] > 10 and res["worst_grad_rel"] < 2e-3, res


def test_sequence_parallel_gather_baseline_matches_serial():
    """The sequence-parallel layouts above run the Ulysses all-to-all baseline (heads divisible by sp); the gather
    baseline (every rank collects all q/k/v rows) must give the same numbers."""
    extra = "wp_topo='(2, 1)', xfmr_wp_topo='(1, 1)', xfmr_sp_size=2, window_assignment_mode='terra_m1_ragged_auto'"
    for res in _run(2, extra, TERRA_SP_BASELINE="gather"):
        assert abs(res["loss"] - res["ref_loss"]) < 1e-4 * max(1.0, abs(res["ref_loss"])), res
        assert res["out_err"] < 2e-3 and res["checked"] > 10 and res["worst_grad_rel"] < 2e-3, res


COLLECTIVES = textwrap.dedent('''
    import json, sys
    sys.path.insert(0, %(root)r)
    import torch, torch.distributed as dist
    from terra_b200.distributed import init_distributed
    from terra_b200.parallel import collectives as C

    rank, world, _ = init_distributed("gloo")
    g = dist.group.WORLD
    torch.manual_seed(rank)
    # ragged all-to-all: rank r sends r + d + 1 rows to rank d
    send = [rank + d + 1 for d in range(world)]
    recv = [s + rank + 1 for s in range(world)]
    x = (torch.arange(sum(send) * 3, dtype=torch.float64).reshape(-1, 3) + 1000 * rank).requires_grad_(True)
    y = C.all_to_all_rows(x, g, send, recv)
    # what must arrive from source s: its chunk for me
    ok = True
    off = 0
    for s in range(world):
        s_send = [s + d + 1 for d in range(world)]
        start = sum(s_send[:rank])
        want = torch.arange(sum(s_send) * 3, dtype=torch.float64).reshape(-1, 3)[start:start + s_send[rank]] + 1000 * s
        ok = ok and torch.equal(y[off:off + recv[s]].detach(), want)
        off += recv[s]
    # adjoint: d/dx sum_r <w_r, y_r> with w_r = (r + 1): the gradient of a row is the weight of the rank it went to
    (y * (rank + 1)).sum().backward()
    want_g = torch.cat([torch.full((send[d], 3), float(d + 1), dtype=torch.float64) for d in range(world)])
    ok = ok and torch.equal(x.grad, want_g)
    # ring: forward one place, gradient comes back one place
    z = torch.full((2,), float(rank), dtype=torch.float64, requires_grad=True)
    got = C.ring_transfer(z, g, 1)
    ok = ok and torch.equal(got.detach(), torch.full((2,), float((rank - 1) %% world), dtype=torch.float64))
    (got * (rank + 10)).sum().backward()
    ok = ok and torch.equal(z.grad, torch.full((2,), float((rank + 1) %% world + 10), dtype=torch.float64))
    print("RESULT " + json.dumps(dict(ok=bool(ok))), flush=True)
    dist.destroy_process_group()
''')


def test_all_to_all_and_ring_transfer_with_their_adjoints():
    for res in _run(3, "", code=COLLECTIVES % dict(root=ROOT)):
        assert res["ok"], res


DIST_MATMUL = textwrap.dedent('''
    import json, sys
    sys.path.insert(0, %(root)r)
    import torch, torch.distributed as dist
    from terra_b200.distributed import init_distributed
    from terra_b200.parallel import dist_matmul as D

    rank, world, _ = init_distributed("gloo")
    g = dist.group.WORLD
    torch.manual_seed(0)                                    # the same full operands on every rank
    T, IN, OUT = 12, 8, 6 * world
    xf = torch.randn(T, IN, dtype=torch.float64)
    wf = torch.randn(OUT, IN, dtype=torch.float64)
    bf = torch.randn(OUT, dtype=torch.float64)
    cot = torch.randn(T, OUT, dtype=torch.float64)          # cotangent of the full output
    xr, wr, br = xf.clone().requires_grad_(True), wf.clone().requires_grad_(True), bf.clone().requires_grad_(True)
    (D.full_reference(xr, wr, br) * cot).sum().backward()
    worst = 0.0
    for isplit in D.LAYOUTS:
        for osplit in D.LAYOUTS:
            x = D.shard(xf, isplit, rank, world).clone().requires_grad_(True)
            wsplit = "(1,n)" if isplit == "(1,n)" else "(m,1)"
            w = D.shard(wf, wsplit, rank, world).clone().requires_grad_(True)
            # the bias is added once per output element: by everybody for column-sharded outputs (own columns), and
            # for row-sharded outputs of a distributed contraction after the reduction (whole bias)
            b = (D.shard(bf[None], "(1,n)", rank, world)[0] if osplit == "(1,n)" else bf).clone().requires_grad_(True)
            y = D.xwt_apply(x, w, b, g, isplit, osplit)
            want = D.shard(D.full_reference(xf, wf, bf), osplit, rank, world)
            worst = max(worst, (y.detach() - want).abs().max().item())
            (y * D.shard(cot, osplit, rank, world)).sum().backward()
            worst = max(worst, (x.grad - D.shard(xr.grad, isplit, rank, world)).abs().max().item())
            worst = max(worst, (w.grad - D.shard(wr.grad, wsplit, rank, world)).abs().max().item())
            gb = b.grad.clone()
            if osplit == "(m,1)":
                dist.all_reduce(gb)                          # every rank saw only its rows
                worst = max(worst, (gb - br.grad).abs().max().item())
            else:
                worst = max(worst, (gb - D.shard(br.grad[None], "(1,n)", rank, world)[0]).abs().max().item())
    print("RESULT " + json.dumps(dict(worst=worst)), flush=True)
    dist.destroy_process_group()
''')


def test_distributed_matmul_layouts_and_gradients():
    """All four (input split, output split) layouts of the distributed X W^T against the undistributed product: the
    output shard, and the shards of the input / weight / bias gradients (reference: core/dist_matmul.py:8-459)."""
    for res in _run(2, "", code=DIST_MATMUL % dict(root=ROOT)):
        assert res["worst"] < 1e-10, res


LEGACY_EMB = textwrap.dedent('''
    import json, sys
    sys.path.insert(0, %(root)r)
    import torch, torch.distributed as dist
    from terra_b200.distributed import init_distributed
    from terra_b200.models.legacy_embeddings import DomainParaPatchEmbedding, DomainParaPatchRecovery
    from terra_b200.parallel.dist_matmul import shard

    rank, world, _ = init_distributed("gloo")
    g = dist.group.WORLD
    worst = 0.0
    for isplit, osplit in (("(1,n)", "(m,1)"), ("(m,1)", "(m,1)"), ("(m,1)", "(1,n)"), ("(1,n)", "(1,n)")):
        torch.manual_seed(3)                                   # every rank draws the same full weights
        full = torch.nn.Linear(4 * 4 * 3, 16)
        torch.manual_seed(3)
        emb = DomainParaPatchEmbedding(g, patch_size=4, num_channel=3, embedding_dim=16, input_split=isplit, output_split=osplit)
        torch.manual_seed(9)
        x = torch.randn(2, 8, 48)
        xs = shard(x.reshape(-1, 48), isplit, rank, world)
        y = emb(xs)
        want = shard(full(x.reshape(-1, 48)), osplit, rank, world)
        worst = max(worst, (y - want).abs().max().item())
    torch.manual_seed(5)
    full = torch.nn.Linear(16, 48)
    torch.manual_seed(5)
    rec = DomainParaPatchRecovery(g, patch_size=4, num_channel=3, embedding_dim=16, input_split="(m,1)", output_split="(1,n)")
    h = torch.randn(16, 16)
    worst = max(worst, (rec(shard(h, "(m,1)", rank, world)) - shard(full(h), "(1,n)", rank, world)).abs().max().item())
    print("RESULT " + json.dumps(dict(worst=worst)), flush=True)
    dist.destroy_process_group()
''')


def test_legacy_domain_parallel_embeddings_match_the_full_linear():
    for res in _run(2, "", code=LEGACY_EMB % dict(root=ROOT)):
        assert res["worst"] < 1e-5, res


DOMAIN_PARALLEL = textwrap.dedent('''
    import copy, json, sys
    sys.path.insert(0, %(root)r)
    import torch, torch.nn as nn, torch.distributed as dist
    from terra_b200.distributed import init_distributed
    from terra_b200.parallel import domain_parallel as DP

    rank, world, _ = init_distributed("gloo")
    dom = DP.DomainGroup(dist.group.WORLD)
    torch.manual_seed(0)
    torch.set_default_dtype(torch.float64)

    class Periodic(nn.Module):                       # circular in W, reflect in H, then an unpadded convolution
        def __init__(self):
            super().__init__()
            self.padding = 1
            self.conv = nn.Conv2d(8, 8, 3, padding=0)
        def forward(self, x):
            x = nn.functional.pad(x, (1, 1, 0, 0), mode="circular")
            return self.conv(nn.functional.pad(x, (0, 0, 1, 1), mode="reflect"))

    full = nn.Sequential(
        nn.Conv2d(3, 8, 3, padding=1), nn.GroupNorm(2, 8), nn.SiLU(),
        nn.Conv2d(8, 8, 3, stride=2, padding=1), nn.Conv2d(8, 8, 1),
        nn.ConvTranspose2d(8, 8, 4, stride=2, padding=1), nn.GroupNorm(4, 8),
        nn.Conv2d(8, 8, 5, padding=2, dilation=1), nn.ConvTranspose2d(8, 4, 2, stride=2))
    par = DP.convert_to_domain_parallel(copy.deepcopy(full), dom)
    counts = par.domain_parallel_counts
    x = torch.randn(2, 3, 16 * world, 12)
    cot = torch.randn(2, 4, 32 * world, 24)
    xr = x.clone().requires_grad_(True)
    yf = full(xr)
    (yf * cot).sum().backward()
    xs = DP.shard_tensor(x, -2, dom).requires_grad_(True)
    yp = par(xs)
    (yp * DP.shard_tensor(cot, -2, dom)).sum().backward()
    worst = (yp.detach() - DP.shard_tensor(yf.detach(), -2, dom)).abs().max().item()
    worst = max(worst, (xs.grad - DP.shard_tensor(xr.grad, -2, dom)).abs().max().item())
    for pf, pp in zip(full.parameters(), par.parameters()):
        g = pp.grad.clone(); dist.all_reduce(g)                  # every rank saw its rows only
        worst = max(worst, (g - pf.grad).abs().max().item())
    gathered = DP.gather_tensor(yp.detach(), -2, dom)
    worst = max(worst, (gathered - yf.detach()).abs().max().item())

    # 3-D layers: [B, C, T, H, W] cut along H
    full3 = nn.Sequential(nn.Conv3d(2, 4, 3, padding=1), nn.ConvTranspose3d(4, 2, (1, 4, 4), stride=(1, 2, 2), padding=(0, 1, 1)))
    par3 = DP.convert_to_domain_parallel(copy.deepcopy(full3), dom)
    v = torch.randn(1, 2, 3, 8 * world, 6)
    worst = max(worst, (par3(DP.shard_tensor(v, 3, dom)) - DP.shard_tensor(full3(v), 3, dom)).abs().max().item())
    counts3 = par3.domain_parallel_counts

    # a custom wrapper replaced as a whole; inner rows agree (the first and the last row differ by design: zero halo
    # at the poles instead of the reflection)
    per = Periodic()
    pper = DP.convert_to_domain_parallel(nn.Sequential(copy.deepcopy(per)), dom,
                                         custom_converters={Periodic: lambda m: DP.DomainParallelPeriodicConv2d(m, dom=dom)})
    u = torch.randn(1, 8, 8 * world, 10)
    a, b = pper(DP.shard_tensor(u, -2, dom)), DP.shard_tensor(per(u), -2, dom)
    lo, hi = (1 if rank == 0 else 0), (a.shape[2] - 1 if rank == world - 1 else a.shape[2])
    worst = max(worst, (a[:, :, lo:hi] - b[:, :, lo:hi]).abs().max().item())

    batch = DP.shard_batch({"x": x, "t": torch.zeros(2), "v": v, "name": "n"}, dom=dom)
    ok = batch["x"].shape[2] == 16 and batch["v"].shape[3] == 8 and batch["t"].shape == (2,) and batch["name"] == "n"
    notes = DP.validate_sharding_constraints(par, 12, window_sizes=[8, (4, 4)])
    print("RESULT " + json.dumps(dict(worst=worst, counts=counts, counts3=counts3, ok=bool(ok), notes=len(notes),
                                      custom=pper.domain_parallel_counts["custom"])), flush=True)
    dist.destroy_process_group()
''')


@pytest.mark.parametrize("world", [2, 3])
def test_generic_domain_parallel_layers_match_the_unsharded_model(world):
    """``convert_to_domain_parallel`` on a stack of plain / strided / wide convolutions, overlapping and non-overlapping
    transposed convolutions and GroupNorms: outputs, input gradients and (summed) parameter gradients of the sharded
    model equal the unsharded one (reference: credit/domain_parallel/*)."""
    for res in _run(world, "", code=DOMAIN_PARALLEL % dict(root=ROOT)):
        assert res["worst"] < 1e-9, res
        assert res["counts"] == {"conv2d": 3, "conv3d": 0, "conv_transpose2d": 1, "conv_transpose3d": 0, "group_norm": 2,
                                 "custom": 0}, res
        assert res["counts3"]["conv3d"] == 1 and res["counts3"]["conv_transpose3d"] == 1 and res["custom"] == 1
        assert res["ok"] and res["notes"] == 2          # 12 % 8 and 6 % 4


TENSOR_PARALLEL = textwrap.dedent('''
    import json, sys
    sys.path.insert(0, %(root)r)
    import torch, torch.nn as nn, torch.nn.functional as F, torch.distributed as dist
    from terra_b200.distributed import init_distributed
    from terra_b200.parallel import tensor_parallel as TP

    rank, world, _ = init_distributed("gloo")
    g = dist.group.WORLD
    torch.set_default_dtype(torch.float64)
    worst = 0.0
    C, Fh, B, S = 8, 8 * world, 2, 4 * world

    def serial(seed):
        torch.manual_seed(seed)
        norm, fc1, fc2 = nn.LayerNorm(C), nn.Linear(C, Fh), nn.Linear(Fh, C)
        return norm, fc1, fc2

    torch.manual_seed(1)
    x = torch.randn(B, S, C)
    cot = torch.randn(B, S, C)
    # ---- Megatron tensor parallel: replicated activations
    torch.manual_seed(5)
    tp = TP.TensorParallelMLP(g, C, Fh)            # draws norm, fc1, fc2 in this order from seed 5
    norm, fc1, fc2 = serial(5)
    xr = x.clone().requires_grad_(True)
    yr = xr + fc2(F.gelu(fc1(norm(xr))))
    (yr * cot).sum().backward()
    xp = x.clone().requires_grad_(True)
    yp = tp(xp)
    (yp * cot).sum().backward()
    per = Fh // world
    worst = max(worst, (yp - yr).abs().max().item(), (xp.grad - xr.grad).abs().max().item())
    worst = max(worst, (tp.weight1.grad - fc1.weight.grad[rank * per:(rank + 1) * per]).abs().max().item())
    worst = max(worst, (tp.weight2.grad - fc2.weight.grad[:, rank * per:(rank + 1) * per]).abs().max().item())
    worst = max(worst, (tp.bias2.grad - fc2.bias.grad).abs().max().item())
    # ---- Megatron sequence parallel: token shards outside the layer
    torch.manual_seed(5)
    sp = TP.MegatronSequenceParallelMLP(g, C, Fh, seq_dim=1)
    sh = S // world
    xs = x[:, rank * sh:(rank + 1) * sh].clone().requires_grad_(True)
    ys = sp(xs)
    (ys * cot[:, rank * sh:(rank + 1) * sh]).sum().backward()
    worst = max(worst, (ys - yr[:, rank * sh:(rank + 1) * sh]).abs().max().item())
    worst = max(worst, (xs.grad - xr.grad[:, rank * sh:(rank + 1) * sh]).abs().max().item())
    worst = max(worst, (sp.weight1.grad - fc1.weight.grad[rank * per:(rank + 1) * per]).abs().max().item())
    gb = sp.bias2.grad.clone(); dist.all_reduce(gb)               # bias2 sees this rank's tokens only
    worst = max(worst, (gb - fc2.bias.grad).abs().max().item())
    # ---- Ulysses: replicated weights, token shards, gradients summed afterwards
    torch.manual_seed(5)
    ul = TP.UlyssesSequenceParallelMLP(C, Fh)
    yu = ul(x[:, rank * sh:(rank + 1) * sh])
    (yu * cot[:, rank * sh:(rank + 1) * sh]).sum().backward()
    gw = ul.fc1.weight.grad.clone(); dist.all_reduce(gw)
    worst = max(worst, (yu - yr[:, rank * sh:(rank + 1) * sh]).abs().max().item(), (gw - fc1.weight.grad).abs().max().item())
    # ---- head <-> token exchange and its inverse, with gradients
    H = 2 * world
    t = torch.randn(B, sh, H, 3, requires_grad=True)              # [B, S / n, heads, d]
    full = TP.all_to_all_dims(t, g, split_dim=2, concat_dim=1)    # [B, S, heads / n, d]
    ok = tuple(full.shape) == (B, S, H // world, 3)
    gathered = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(gathered, t.detach())
    want = torch.cat(gathered, dim=1)[:, :, rank * 2:(rank + 1) * 2]
    worst = max(worst, (full.detach() - want).abs().max().item())
    back = TP.all_to_all_dims(full, g, split_dim=1, concat_dim=2)
    worst = max(worst, (back.detach() - t.detach()).abs().max().item())
    (back * 3.0).sum().backward()
    worst = max(worst, (t.grad - 3.0).abs().max().item())
    # ---- last-dimension regions
    z = torch.randn(3, 4 * world, requires_grad=True)
    piece = TP.scatter_to_region(z, g)
    again = TP.gather_from_region(piece, g)
    worst = max(worst, (again.detach() - z.detach()).abs().max().item())
    (again * (rank + 1.0)).sum().backward()
    # gather's adjoint keeps this rank's slice of the cotangent, scatter's adjoint gathers the slices of all ranks:
    # slice j of the input gradient is rank j's weight
    wantg = torch.cat([torch.full((3, 4), r + 1.0) for r in range(world)], dim=-1)
    worst = max(worst, (z.grad - wantg).abs().max().item())
    print("RESULT " + json.dumps(dict(worst=worst, ok=bool(ok))), flush=True)
    dist.destroy_process_group()
''')


def test_classic_tensor_and_sequence_parallel_layers_match_the_serial_mlp():
    """Megatron tensor-parallel, Megatron sequence-parallel and Ulysses MLPs over a 2-rank group against the serial MLP
    with the same seeded weights (outputs, input gradients, weight-shard gradients), plus the head <-> token all-to-all
    and the last-dimension scatter / gather regions (reference: core/tensor_parallel.py, models/mlp.py:177-373)."""
    for res in _run(2, "", code=TENSOR_PARALLEL % dict(root=ROOT)):
        assert res["ok"] and res["worst"] < 1e-10, res
