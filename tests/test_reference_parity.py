"""The CPU fp32 build against the reference's own ``SequentialHierarchicalSwin`` (installed under ``baseline/_ref``):
same ``state_dict`` keys and shapes, bit-identical initial weights (the seeded construction order is part of the
compatibility contract), same output and gradients, and a reference ``state_dict`` loads. Skipped when the reference
is not installed."""
import pytest
import torch

from baseline import ref_import

pytestmark = pytest.mark.skipif(not ref_import.available(), reason="reference is not installed under baseline/_ref")

KW = dict(padding_scale=2, num_channels=64, patch_size=4, window_size=8, height=128, width=256, embedding_dim=96,
          num_heads=3, num_layers=2)


def _build_both(seed=1234, **over):
    ref_import.enable()
    from models.reference_model.sequential_hierarchical_swin import SequentialHierarchicalSwin as RefSeq   # reference

    from terra_b200.models import SequentialHierarchicalSwin

    kw = dict(KW, **over)
    torch.manual_seed(seed)
    ref = RefSeq(**kw)
    torch.manual_seed(seed)
    mine = SequentialHierarchicalSwin(**kw)
    return ref, mine


def test_state_dict_keys_shapes_and_initial_weights_are_identical():
    ref, mine = _build_both()
    sd_ref, sd = ref.state_dict(), mine.state_dict()
    # the reference materialises the shift mask as a buffer; here it is derived inside the attention kernel
    ref_keys = {k for k in sd_ref if not k.endswith("attn_mask")}
    assert ref_keys == set(sd), (sorted(ref_keys - set(sd)), sorted(set(sd) - ref_keys))
    for k in sd:
        assert tuple(sd[k].shape) == tuple(sd_ref[k].shape), k
        assert torch.equal(sd[k].float(), sd_ref[k].float()), f"initial value of {k} differs"


def test_forward_and_gradients_match_the_reference():
    ref, mine = _build_both()
    torch.manual_seed(7)
    x = torch.randn(1, KW["height"], KW["width"], KW["num_channels"])
    yr, ym = ref(x), mine(x)
    assert (yr - ym).abs().max().item() <= 2e-4 * max(1.0, yr.abs().max().item())
    (yr - x).abs().mean().backward()
    (ym - x).abs().mean().backward()
    gr, gm = dict(ref.named_parameters()), dict(mine.named_parameters())
    for k, p in gm.items():
        a, b = p.grad, gr[k].grad
        assert (a - b).abs().max().item() <= 1e-3 * (b.abs().max().item() + 1e-9) + 1e-8, k


def test_reference_state_dict_loads_and_reproduces_its_output():
    ref, mine = _build_both()
    with torch.no_grad():
        for p in ref.parameters():
            p.add_(0.01 * torch.randn_like(p))
    missing = mine.load_state_dict(ref.state_dict(), strict=True)      # attn_mask entries are dropped on load
    assert not missing.missing_keys and not missing.unexpected_keys
    x = torch.randn(1, KW["height"], KW["width"], KW["num_channels"])
    with torch.no_grad():
        assert (ref(x) - mine(x)).abs().max().item() <= 2e-4 * max(1.0, float(ref(x).abs().max()))


def test_unshifted_only_model_and_no_bias_variant_match():
    ref, mine = _build_both(num_layers=1)
    x = torch.randn(1, KW["height"], KW["width"], KW["num_channels"])
    with torch.no_grad():
        assert (ref(x) - mine(x)).abs().max().item() <= 2e-4 * max(1.0, float(ref(x).abs().max()))


def test_window_utilities_match_the_reference_and_the_kernel_index_math():
    """``ops/window_utils.py`` against the reference's helpers (models/utils.py), and against the closed-form region
    numbering that the attention kernels use instead of a mask tensor."""
    import models.utils as ref_utils

    from terra_b200.ops import window_utils as U
    from terra_b200.ops.attention import region_ids

    torch.manual_seed(0)
    x = torch.randn(2, 16, 24, 5)
    assert torch.equal(U.window_partition(x, 8), ref_utils.window_partition(x, 8))
    assert torch.equal(U.window_reverse(U.window_partition(x, 8), 8, 16, 24), x)
    assert torch.equal(U.window_reverse(ref_utils.window_partition(x, 8), 8, 16, 24),
                       ref_utils.window_reverse(ref_utils.window_partition(x, 8), 8, 16, 24))
    h = torch.randn(16, 24, 2, 5)
    assert torch.equal(U.window_partition_HWBC(h, 8), ref_utils.window_partition_HWBC(h, 8))
    for res, win in (((13, 721, 1440), (2, 6, 12)), ((4, 48, 96), (2, 6, 12)), ((7, 50, 99), (3, 8, 8))):
        assert tuple(U.get_pad3d(res, win)) == tuple(ref_utils.get_pad3d(res, win))
        assert tuple(U.get_pad2d(res[1:], win[1:])) == tuple(ref_utils.get_pad2d(res[1:], win[1:]))
    mask = U.get_swin_attention_mask("sequential", (16, 24), 8, 4)
    assert torch.equal(mask, ref_utils.get_swin_attention_mask("sequential", (16, 24), 8, 4))
    # the kernels' closed form: region numbers of the rolled frame, rectangular windows included
    for (H, W, wh, ww) in ((16, 24, 8, 8), (16, 36, 8, 12)):
        want = U.shift_region_map(H, W, (wh, ww), (wh // 2, ww // 2))
        assert torch.equal(region_ids(H, W, wh, ww, wh // 2, ww // 2).reshape(H, W).long(), want)
