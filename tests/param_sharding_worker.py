"""Worker of tests/test_param_sharding_cpu.py: run as gloo ranks under torch.distributed.run.

A small stack of residual blocks is trained with sharded parameters on every rank's own data; rank 0 compares with one
process that holds the whole model, sums the ranks' losses and steps ``torch.optim.AdamW``.
"""
import json
import os
import sys

import torch
import torch.distributed as dist
from torch.utils.checkpoint import checkpoint

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from terra_b200.optim.sharded_param_adamw import ShardedParamAdamW  # noqa: E402
from terra_b200.parallel.param_sharding import ParamSharder  # noqa: E402


class Block(torch.nn.Module):
    def __init__(self, d):
        super().__init__()
        self.norm = torch.nn.LayerNorm(d)
        self.fc1 = torch.nn.Linear(d, 2 * d)
        self.fc2 = torch.nn.Linear(2 * d, d)
        self.table = torch.nn.Parameter(torch.zeros(d))          # a parameter on a branch of its own

    def forward(self, x):
        return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.norm(x)))) + self.table[torch.arange(x.shape[-1])]


class Layer(torch.nn.Module):
    def __init__(self, d, depth, recompute):
        super().__init__()
        self.blocks = torch.nn.ModuleList([Block(d) for _ in range(depth)])
        self.recompute = recompute

    def run(self, s, e, x):
        for i in range(s, e):
            x = self.blocks[i](x)
        return x

    def forward(self, x):
        if not self.recompute:
            return self.run(0, len(self.blocks), x)
        half = len(self.blocks) // 2
        x = checkpoint(lambda t: self.run(0, half, t), x, use_reentrant=False)
        return self.run(half, len(self.blocks), x)


class Net(torch.nn.Module):
    def __init__(self, d=24, depth=4, recompute=False):
        super().__init__()
        self.embed = torch.nn.Linear(8, d)
        self.layer = Layer(d, depth, recompute)
        self.head = torch.nn.Linear(d, 8)

    def forward(self, x):
        return self.head(self.layer(self.embed(x)))


def data(rank, step, rollout):
    g = torch.Generator().manual_seed(1000 * step + rank)
    return [torch.randn(6, 8, generator=g) for _ in range(rollout)], torch.randn(6, 8, generator=g)


def loss_of(net, xs, y):
    # rollout > 1: several forward passes before the one backward pass
    out = xs[0]
    total = 0.0
    for i, x in enumerate(xs):
        out = net(x + (0.1 * out.detach() if i else 0.0))
        total = total + torch.nn.functional.mse_loss(out, y)
    return total


def working_copy_mode(rank, world):
    """The bookkeeping of the GPU form on CPU tensors: a bf16 working copy is what gets gathered, the fp32 values exist
    only under ``summon_full_params``. No model compute (the CPU operators read the fp32 values): gradients are
    written by hand, the way the GPU kernels write them into the gradient views."""
    torch.manual_seed(7)
    net, ref = Net(), Net()
    ref.load_state_dict(net.state_dict())
    group = dist.group.WORLD
    sharder = ParamSharder(net, lambda label: (group, rank, world), bf16_shadow=True)
    opt = ShardedParamAdamW(sharder, lr=1e-2, weight_decay=0.1)
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    assert sharder.resident_bytes() == 0
    names = dict(net.named_parameters())
    for step in range(3):
        opt.zero_grad()
        for u in sharder.all_units():
            u.gather()
            assert u.arena.master.untyped_storage().size() == 0, "the fp32 values stay released"
            for p in u.params:
                n = [k for k, v in names.items() if v is p][0]
                want = dict(ref.named_parameters())[n].detach()
                # bf16 of this optimizer's fp32 values; the oracle's differ in the last fp32 bits, which may move a
                # bf16 rounding: one bf16 step of slack
                assert p.bf16.dtype == torch.bfloat16 and p.bf16.shape == want.shape
                assert ((p.bf16.float() - want).abs() <= want.abs() * 2 ** -7 + 1e-30).all(), (step, n)
                assert getattr(p, "terra_master_sharded", False)
            u.materialise_grad()
            for i, p in enumerate(u.params):
                p.grad.fill_(0.01 * (rank + 1) * (i + 1) * (step + 1))
            u.reduce_grad()
            u.release()
        opt.step()
        for i_all, (n, q) in enumerate(ref.named_parameters()):
            unit = [u for u in sharder.all_units() if any(x is names[n] for x in u.params)][0]
            i = [k for k, x in enumerate(unit.params) if x is names[n]][0]
            q.grad = torch.full_like(q, sum(0.01 * (r + 1) * (i + 1) * (step + 1) for r in range(world)))
        ref_opt.step()
    got = sharder.full_state_dict()
    err = max((got[k] - v).abs().max().item() for k, v in ref.state_dict().items())
    assert err < 1e-6, err
    assert sharder.resident_bytes() == 0
    if rank == 0:
        print("RESULT " + json.dumps(dict(worst=err)), flush=True)


def main():
    mode = json.loads(sys.argv[1])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    if mode.get("working_copy"):
        working_copy_mode(rank, world)
        dist.barrier()
        dist.destroy_process_group()
        return
    torch.manual_seed(7)
    net = Net(recompute=mode.get("recompute", False))
    ref = Net(recompute=False)
    ref.load_state_dict(net.state_dict())
    total = sum(p.numel() for p in net.parameters())

    group = dist.group.WORLD
    sharder = ParamSharder(net, lambda label: (group, rank, world), blocks_per_unit=mode.get("blocks_per_unit", 1),
                           whole_model=mode.get("whole_model", False), prefetch=mode.get("prefetch", "none"),
                           reshard_after_forward=mode.get("reshard_after_forward", True))
    opt = ShardedParamAdamW(sharder, lr=1e-2, weight_decay=0.1)
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    assert sharder.resident_bytes() == 0, "nothing but the owned slices exists between steps"
    assert sharder.owned_numel() * world == sharder.total_numel() >= total

    from terra_b200.runtime.grad_debug import report_unit_gradients
    observed, lines = [], []
    sharder.observe_gradients(lambda u: (observed.append(u.name), report_unit_gradients(u, limit=10 ** 9, printer=lines.append)))
    peak = [0]

    def watch(mod, args):
        peak[0] = max(peak[0], sharder.resident_bytes())
    for b in net.layer.blocks:
        b.register_forward_pre_hook(watch)

    rollout = mode.get("rollout", 1)
    worst = 0.0
    for step in range(4):
        opt.zero_grad()
        xs, y = data(rank, step, rollout)
        loss = loss_of(net, xs, y)
        loss.backward()
        if mode.get("clip"):
            norm = opt.clip_grad_norm_(0.5)
        opt.step()
        assert sharder.resident_bytes() == 0

        ref_opt.zero_grad()
        ref_loss = 0.0
        for r in range(world):
            xr, yr = data(r, step, rollout)
            ref_loss = ref_loss + loss_of(ref, xr, yr)
        ref_loss.backward()
        if mode.get("clip"):
            ref_norm = float(torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5))
            assert abs(norm - ref_norm) <= 1e-4 * ref_norm, (norm, ref_norm)
        ref_opt.step()
        both = loss.detach().clone()
        dist.all_reduce(both)
        worst = max(worst, abs(both.item() - ref_loss.item()) / abs(ref_loss.item()))
    assert worst < 1e-5, worst

    got = sharder.full_state_dict()
    err = max((got[k] - v).abs().max().item() for k, v in ref.state_dict().items())
    assert err < 1e-5, err

    # the gathered optimizer state is torch.optim.AdamW's
    full = opt.full_state_dict()
    want = ref_opt.state_dict()["state"]
    assert set(full["state"]) == set(want)
    for i, st in want.items():
        assert (full["state"][i]["exp_avg"] - st["exp_avg"]).abs().max().item() < 1e-5
        assert (full["state"][i]["exp_avg_sq"] - st["exp_avg_sq"]).abs().max().item() < 1e-6
        assert float(full["state"][i]["step"]) == float(st["step"])

    # both checkpoint forms restore the run: the per-rank slices, and the gathered form into a fresh layout
    own = opt.state_dict()
    net2 = Net(recompute=mode.get("recompute", False))
    sharder2 = ParamSharder(net2, lambda label: (group, rank, world), blocks_per_unit=2, prefetch="none")
    opt2 = ShardedParamAdamW(sharder2, lr=1e-2, weight_decay=0.1)
    sharder2.load_full_state_dict(got)
    opt2.load_state_dict(full)
    opt.load_state_dict(own)
    xs, y = data(rank, 99, rollout)
    losses = []
    for n, o in ((net, opt), (net2, opt2)):
        o.zero_grad()
        loss_of(n, xs, y).backward()
        o.step()
        with torch.no_grad():
            losses.append(float(loss_of(n, xs, y)))
    assert abs(losses[0] - losses[1]) <= 1e-5 * abs(losses[0]), losses

    units = sharder.all_units()
    if rank == 0:
        print("RESULT " + json.dumps(dict(
            worst=worst, total_bytes=4 * sharder.total_numel(), peak_bytes=peak[0], units=len(sharder.units),
            gathers=[u.gathers for u in units], reductions=[u.reductions for u in units], observed=len(observed),
            lines=len(lines), first_line=lines[0])), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
