"""Step-runtime helpers that need no GPU."""
import torch


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
