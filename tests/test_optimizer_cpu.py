"""Optimizer semantics on the CPU: the sharded ``DistributedAdamW`` on gloo ranks against ``torch.optim.AdamW`` over
several steps, its checkpoint round trip, and the dynamic loss scaler."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys, json, io
    sys.path.insert(0, %(root)r)
    import torch, torch.distributed as dist
    from terra_b200.optim.distributed_adamw import DistributedAdamW
    from terra_b200.utils.flat_params import ParamArena

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", init_method="env://", rank=rank, world_size=world)

    def make():
        torch.manual_seed(3)
        return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.GELU(), torch.nn.Linear(40, 24), torch.nn.LayerNorm(24))

    mine, ref = make(), make()
    ParamArena(mine)
    opt = DistributedAdamW(mine.parameters(), lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, model=mine,
                           process_group=dist.group.WORLD)
    ropt = torch.optim.AdamW(ref.parameters(), lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    worst = 0.0
    for step in range(6):
        if step == 3:
            # checkpoint round trip in the middle: a fresh optimizer loaded from the state continues identically
            buf = io.BytesIO(); torch.save(opt.state_dict(), buf); buf.seek(0)
            opt2 = DistributedAdamW(mine.parameters(), lr=1.0, model=mine, process_group=dist.group.WORLD)
            opt2.load_state_dict(torch.load(buf, weights_only=False))
            opt = opt2
        opt.zero_grad(); ropt.zero_grad()
        # every rank sees its own data; the reference model sees all of it (sum of the ranks' losses)
        total = 0.0
        for r in range(world):
            g = torch.Generator().manual_seed(100 * step + r)
            x = torch.randn(8, 24, generator=g)
            if r == rank:
                mine(x).square().mean().backward()
            total = total + ref(x).square().mean()
        total.backward()
        opt.step(); ropt.step()
        for p, q in zip(mine.parameters(), ref.parameters()):
            worst = max(worst, (p.data - q.data).abs().max().item())
    # per-parameter view of the sharded state == torch.optim.AdamW's own state, and torch's state loads back in
    full = opt.full_state_dict()
    rstate = ropt.state_dict()["state"]
    state_err = max(max((full["state"][i]["exp_avg"] - rstate[i]["exp_avg"]).abs().max().item(),
                        (full["state"][i]["exp_avg_sq"] - rstate[i]["exp_avg_sq"]).abs().max().item()) for i in rstate)
    opt3 = DistributedAdamW(mine.parameters(), lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, model=mine,
                            process_group=dist.group.WORLD)
    opt3.load_state_dict(ropt.state_dict())
    round_trip = max((a.exp_avg[:a.hi - a.lo] - b.exp_avg[:b.hi - b.lo]).abs().max().item()
                     for a, b in zip(opt3.shards, opt.shards) if a.hi > a.lo)
    assert opt3.step_count == opt.step_count
    owned = sum(s.hi - s.lo for s in opt.shards)
    with open(os.path.join(os.environ["OUT_DIR"], f"res_{rank}.json"), "w") as f:      # (stdout of ranks interleaves)
        json.dump(dict(rank=rank, worst=worst, owned=owned, numel=opt.arena.numel, state_err=state_err, round_trip=round_trip), f)
    dist.destroy_process_group()
''')


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world", [2, 3])
def test_distributed_adamw_equals_torch_adamw_over_steps(tmp_path, world):
    import json

    script = tmp_path / "w.py"
    script.write_text(WORKER % dict(root=ROOT))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1", OUT_DIR=str(tmp_path))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script)],
                         env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-4000:])
    res = [json.load(open(tmp_path / f"res_{r}.json")) for r in range(world)]
    for r in res:
        assert r["worst"] < 3e-5, r                      # same update rule in fp32; the ranks' gradients are summed in another order
        assert 0 < r["owned"] <= r["numel"]              # every rank owns a slice, none owns everything (world > 1)
        assert r["state_err"] < 3e-5 and r["round_trip"] < 3e-5, r
    assert sum(r["owned"] for r in res) >= res[0]["numel"] - 1024 * world


def test_loss_scaler_skips_on_overflow_backs_off_and_grows():
    from terra_b200.optim.grad_scaler import LossScaler

    class Opt:
        def __init__(self):
            self.calls = []

        def step(self, grad_scale=1.0):
            self.calls.append(grad_scale)

    s = LossScaler(init_scale=1024.0, growth_interval=2)
    opt = Opt()
    g = torch.full((100,), 2.0) * 1024.0                     # gradients of the scaled loss: norm / scale = 20
    assert s.step(opt, g, clip_max_norm=1.0) is True
    s.update()
    assert abs(opt.calls[0] - (1 / 1024.0) * (1.0 / 20.0)) < 1e-8       # un-scaling and clipping folded into one factor
    g[7] = float("inf")
    assert s.step(opt, g) is False and len(opt.calls) == 1     # overflow: no optimizer step
    s.update()
    assert s.get_scale() == 512.0 and s.skipped_steps == 1
    g[7] = 1.0
    for _ in range(2):
        assert s.step(opt, g) is True
        s.update()
    assert s.get_scale() == 1024.0                            # two clean steps = growth_interval
    t = LossScaler()
    t.load_state_dict(s.state_dict())
    assert t.get_scale() == 1024.0 and set(s.state_dict()) == {"scale", "growth_factor", "backoff_factor",
                                                               "growth_interval", "_growth_tracker"}


def test_precision_is_never_switched_silently():
    from terra_b200.models.get_model import get_model_for_train

    with pytest.raises(ValueError, match="precision"):
        get_model_for_train({}, {"precision": "fp8", "model_architecture": "nope"})


def test_fp32_reads_take_the_working_copy_when_masters_are_sharded():
    """A kernel that reads a parameter in fp32 (the relative-position bias table) must not read the fp32 master on a
    rank that does not own it: under a sharded optimizer only the bf16 working copy is refreshed everywhere. The
    widened copy is built once per optimizer step."""
    import torch

    from terra_b200.ops.packed import fp32_values, invalidate_packed_weights

    p = torch.nn.Parameter(torch.full((4,), 1.0))
    assert fp32_values(p).data_ptr() == p.data.data_ptr()                    # plain parameter: the master itself
    p.bf16 = torch.full((4,), 2.0, dtype=torch.bfloat16)
    assert fp32_values(p).data_ptr() == p.data.data_ptr()                    # replicated masters are exact everywhere
    p.terra_master_sharded = True
    a = fp32_values(p)
    assert a.dtype == torch.float32 and a.tolist() == [2.0] * 4              # the gathered working copy, widened
    assert fp32_values(p) is a                                               # cached within the step
    p.bf16.fill_(3.0)
    invalidate_packed_weights()                                              # what every optimizer step does
    assert fp32_values(p).tolist() == [3.0] * 4


def test_differentiable_fp32_reads_pass_the_gradient_to_the_parameter():
    """``fp32_param``: PyTorch code that indexes the bias table gets the widened working copy when the fp32 master is
    owner-only, and the table's gradient still arrives at the parameter."""
    import torch

    from terra_b200.ops.packed import fp32_param, invalidate_packed_weights

    p = torch.nn.Parameter(torch.full((5,), 1.0))
    assert fp32_param(p) is p
    p.bf16 = torch.arange(5, dtype=torch.float32).bfloat16()
    p.terra_master_sharded = True
    invalidate_packed_weights()
    t = fp32_param(p)
    assert t is not p and t.dtype == torch.float32 and t.tolist() == [0.0, 1.0, 2.0, 3.0, 4.0] and t.requires_grad
    (t[torch.tensor([1, 1, 3])] * torch.tensor([1.0, 2.0, 5.0])).sum().backward()
    assert p.grad.tolist() == [0.0, 3.0, 0.0, 5.0, 0.0]
    # two uses in one graph are two nodes over fresh tensors
    a, b = fp32_param(p), fp32_param(p)
    assert a is not b
    p.grad = None
    (a.sum() + 2 * b.sum()).backward()
    assert p.grad.tolist() == [3.0] * 5
