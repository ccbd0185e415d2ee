"""Whole-model parity: the CUDA (bf16, sm_100a kernels) build against the CPU fp32 build of the same weights."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

KW = dict(padding_scale=2, num_channels=64, patch_size=4, window_size=8, height=128, width=256, embedding_dim=96,
          num_heads=3, num_layers=2)


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def test_serial_model_forward_backward_matches_cpu():
    from terra_b200.models import SequentialHierarchicalSwin
    from terra_b200.ops.gemm import check_status
    from terra_b200.ops.loss import masked_loss

    torch.manual_seed(0)
    cpu = SequentialHierarchicalSwin(**KW)
    gpu = copy.deepcopy(cpu).cuda()
    x = torch.randn(1, 128, 256, 64)
    label = torch.randn(1, 128, 256, 64)
    mask = (torch.rand(128, 256, 64) > 0.3).float()

    y_cpu = cpu(x)
    loss_cpu = masked_loss(y_cpu, label, mask, "L1")
    loss_cpu.backward()

    y_gpu = gpu(x.cuda())
    loss_gpu = masked_loss(y_gpu, label.cuda().bfloat16(), mask.cuda(), "L1")
    loss_gpu.backward()
    check_status("cuda")

    assert _rel(y_gpu, y_cpu) < 2e-2
    assert abs(loss_gpu.item() - loss_cpu.item()) < 2e-2 * abs(loss_cpu.item())
    gp = dict(gpu.named_parameters())
    bad = []
    for name, p in cpu.named_parameters():
        if p.grad is None or p.grad.norm() < 1e-7:
            continue
        r = _rel(gp[name].grad, p.grad)
        # bf16 activations carry 2^-9 relative rounding per operation; through ~20 dependent kernels (2 blocks, the
        # two sampling stacks, both projections) and the reductions over 2048 tokens the gradients of the CPU fp32
        # and the CUDA bf16 build agree to 2-3 % in norm; the parameters in front of the softmax (q / k projections,
        # bias table) measure 4.5-4.7 %, because the probabilities and their gradients are rounded to bf16 before the
        # products. Sign errors or a wrong scale would show as >= 100 %.
        if r > 0.06:
            bad.append((name, r))
    assert not bad, bad


def test_training_loss_decreases():
    from terra_b200.models import SequentialHierarchicalSwin
    from terra_b200.ops.loss import masked_loss
    from terra_b200.optim import FusedAdamW

    torch.manual_seed(0)
    model = SequentialHierarchicalSwin(**KW).cuda()
    x = torch.randn(1, 128, 256, 64, device="cuda")
    label = x + 0.1 * torch.randn_like(x)
    model(x)   # builds the arena
    opt = FusedAdamW(model.parameters(), lr=1e-3, model=model)
    losses = []
    for _ in range(8):
        opt.zero_grad()
        loss = masked_loss(model(x), label.bfloat16(), None, "L2")
        loss.backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0], losses


def test_loss_curve_follows_the_cpu_fp32_oracle_for_20_steps():
    """Same seeded weights, same data, same optimizer hyper-parameters: the bf16 CUDA build and the fp32 CPU build of
    the model must trace the same loss curve (the acceptance criterion the reference uses for its parallel builds:
    tests/distributed/correctness/analyze_correctness.py:210-241)."""
    from terra_b200.models import SequentialHierarchicalSwin
    from terra_b200.ops.gemm import check_status
    from terra_b200.ops.loss import masked_loss
    from terra_b200.optim import FusedAdamW

    torch.manual_seed(0)
    cpu = SequentialHierarchicalSwin(**KW)
    gpu = copy.deepcopy(cpu).cuda()
    xs = [torch.randn(1, 128, 256, 64) for _ in range(2)]
    ys = [x + 0.3 * torch.randn_like(x) for x in xs]
    gpu(xs[0].cuda())        # builds the flat arena
    opt_g = FusedAdamW(gpu.parameters(), lr=1e-3, model=gpu)
    opt_c = torch.optim.AdamW(cpu.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    curve_c, curve_g = [], []
    for step in range(20):
        x, y = xs[step % 2], ys[step % 2]
        opt_c.zero_grad()
        lc = masked_loss(cpu(x), y, None, "L1")
        lc.backward()
        opt_c.step()
        opt_g.zero_grad()
        lg = masked_loss(gpu(x.cuda()), y.cuda().bfloat16(), None, "L1")
        lg.backward()
        opt_g.step()
        curve_c.append(lc.item())
        curve_g.append(lg.item())
    check_status("cuda")
    assert curve_c[-1] < 0.9 * curve_c[0], curve_c          # the run does train
    for a, b in zip(curve_g, curve_c):
        assert abs(a - b) <= 1.5e-2 * abs(b), (curve_g, curve_c)
