"""Grid padding rules.

``get_padded_shape`` reproduces the reference rule (utils.py:94-119): with an explicit ``padded_shape`` the
extra rows/columns are split ``pad // 2`` before and the rest after; otherwise each dimension is padded up to a
multiple of ``patch_size * padding_scale * window`` (window may differ per dimension here).
``compute_auto_padded_shape`` restates the ``padding_policy: auto`` search of the reference
(models/model_utils/get_model.py:454-585) for rectangular windows.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple


def _pair(v) -> Tuple[int, int]:
    if isinstance(v, (tuple, list)):
        return int(v[0]), int(v[1])
    return int(v), int(v)


def _split_pad(total: int) -> Tuple[int, int]:
    first = total // 2
    return first, total - first


def get_padded_shape(height, width, patch_size, window_size, padding_scale=2, padded_shape=None, downsample=1):
    """Returns ``(need_padding, (left, right, top, bottom), (padded_h, padded_w))``."""
    wh, ww = _pair(window_size)
    if padded_shape is not None:
        ph, pw = (int(v) for v in tuple(padded_shape))
        if ph < height or pw < width:
            raise ValueError(f"padded_shape={padded_shape} must cover input shape={(height, width)}")
        top, bottom = _split_pad(ph - height)
        left, right = _split_pad(pw - width)
    else:
        unit_h = patch_size * padding_scale * wh
        unit_w = patch_size * padding_scale * ww
        top, bottom = _split_pad((-height) % unit_h)
        left, right = _split_pad((-width) % unit_w)
    padded = (height + top + bottom, width + left + right)
    return (left + right + top + bottom) > 0, (left, right, top, bottom), padded


def _ceil_to(v: int, m: int) -> int:
    if m <= 0:
        raise ValueError(f"multiple must be positive, got {m}")
    return -(-v // m) * m


def _lcm(a: int, b: int) -> int:
    return abs(a * b) // math.gcd(a, b)


def _grow_for_total(nh, nw, mh, mw, need):
    """Grow the cheaper dimension (in window multiples) until there are at least ``need`` windows."""
    while nh * nw < need:
        cand_h, cand_w = _ceil_to(nh + 1, mh), _ceil_to(nw + 1, mw)
        if cand_h * nw <= nh * cand_w:
            nh = cand_h
        else:
            nw = cand_w
    return nh, nw


def compute_auto_padded_shape(height, width, patch_size, window_size, downsample, wp_topo, xfmr_wp_topo,
                              window_assignment_mode):
    from ..parallel.window_assignment import is_terra_m1_assignment_mode

    wh, ww = _pair(window_size)
    unit_h, unit_w = patch_size * downsample * wh, patch_size * downsample * ww
    nh, nw = -(-height // unit_h), -(-width // unit_w)
    # token rows must split evenly over the data topology
    mh = wp_topo[0] // math.gcd(wh, wp_topo[0])
    mw = wp_topo[1] // math.gcd(ww, wp_topo[1])
    m, n = xfmr_wp_topo
    mode = window_assignment_mode
    if is_terra_m1_assignment_mode(mode):
        if n != 1:
            raise ValueError(f"{mode} requires xfmr_wp_topo=(m, 1), got xfmr_wp_topo={xfmr_wp_topo}")
        nh, nw = _ceil_to(nh, mh), _ceil_to(nw, mw)
        if mode == "terra_m1_regular":
            nh = _ceil_to(nh, _lcm(mh, m))
        elif mode == "terra_m1_ragged_row":
            nh = max(nh, _ceil_to(m, mh))
        elif mode == "terra_m1_ragged_row_major":
            nh, nw = _grow_for_total(nh, nw, mh, mw, m)
        elif nh < m:                                     # terra_m1_ragged_auto
            nh, nw = _grow_for_total(nh, nw, mh, mw, m)
    elif mode == "regular":
        nh, nw = _ceil_to(nh, _lcm(mh, m)), _ceil_to(nw, _lcm(mw, n))
    elif mode == "ragged_round_robin":
        if tuple(wp_topo) == tuple(xfmr_wp_topo) and wp_topo[1] > 1:
            raise ValueError("auto padding for ragged_round_robin requires data wp_topo=(m, 1) when transformer "
                             f"topology has n > 1, got wp_topo={wp_topo}, xfmr_wp_topo={xfmr_wp_topo}")
        nh, nw = _ceil_to(nh, mh), _ceil_to(nw, mw)
        if n == 1:
            nh = max(nh, m)
        else:
            while nh * nw < m * n:
                cand_h, cand_w = _ceil_to(nh + 1, mh), _ceil_to(nw + 1, mw)
                if (cand_h * unit_h) * (nw * unit_w) <= (nh * unit_h) * (cand_w * unit_w):
                    nh = cand_h
                else:
                    nw = cand_w
    else:
        raise ValueError(f"Unsupported window_assignment_mode={mode}")
    return nh * unit_h, nw * unit_w
