"""Building blocks with the reference's parameter names and initialisation order.

Sequential / window-parallel build (reference: models/attention.py:175-283, models/mlp.py:138-174,375-412,
models/transformer.py:71-135,606-1042, models/reference_model/parallel_layers.py:27-312):

    layers.blocks.{i}.0.norm1, .attn.{relative_position_bias_table, relative_position_index,
                                       q_linear, k_linear, v_linear, proj}
    layers.blocks.{i}.1.norm2, .fc1, .fc2

Factorised SP/TP build (models/attention.py:612-757, models/mlp.py:415-469): q/k/v column-sharded over TP,
``proj`` row-sharded without bias plus a replicated ``attn.proj_bias``; with TP > 1 the MLP is
``linear1`` (column-sharded) / ``linear2`` (row-sharded, no bias) / ``bias2``; the bias table is sharded by
heads. Sharded parameters carry ``terra_grad_reduce_group = "xfmr_tp_param_group"``.

None of these modules has a ``forward`` that moves data around: the math lives in ``terra_b200.ops`` and the
activation layout (window-major, unshifted) is owned by the parallel context.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ..memory.activation import activation_checkpoint
from ..memory.selective_recompute import SelectiveRecomputeScheduler
from ..ops import blocks as B
from ..ops.attention import relative_position_index
from ..ops.packed import fp32_param
from ..profiler.memory_timeline import mark_memory_timeline
from .init_utils import (linear_from_tensors, make_linear_with_seed, run_with_seed, sharded_linear_tensors)

TP_LABEL = "xfmr_tp_param_group"


def to_2tuple(v) -> Tuple[int, int]:
    if isinstance(v, (tuple, list)):
        return int(v[0]), int(v[1])
    return int(v), int(v)


def _tag(module: nn.Module, label: str) -> None:
    for p in module.parameters():
        p.terra_grad_reduce_group = label


class WindowAttention(nn.Module):
    """Parameters of one window-attention layer (optionally the TP shard of it)."""

    _fused_param_groups = {
        "qkv_weight": ["q_linear.weight", "k_linear.weight", "v_linear.weight"],
        "qkv_bias": ["q_linear.bias", "k_linear.bias", "v_linear.bias"],
    }

    def __init__(self, embedding_dim, window_size, num_heads, use_relative_position_bias=True, init_seed_base=None,
                 factorized=False, tp_size=1, tp_rank=0):
        super().__init__()
        self.dim = embedding_dim
        self.window_size = to_2tuple(window_size)
        self.total_heads = num_heads
        if embedding_dim % num_heads != 0:
            raise ValueError(f"dim {embedding_dim} must be divisible by num_heads {num_heads}")
        if num_heads % tp_size != 0 or embedding_dim % tp_size != 0:
            raise ValueError(f"num_heads {num_heads} / dim {embedding_dim} must be divisible by tensor_parallel_size {tp_size}")
        self.num_heads = num_heads // tp_size                 # heads held by this rank
        self.local_dim = embedding_dim // tp_size
        self.scale = (embedding_dim // num_heads) ** -0.5
        self.use_relative_position_bias = use_relative_position_bias
        self.factorized = factorized
        wh, ww = self.window_size
        seed = (lambda k: None if init_seed_base is None else init_seed_base + k)

        if use_relative_position_bias:
            table = torch.zeros((2 * wh - 1) * (2 * ww - 1), num_heads)
            run_with_seed(init_seed_base, lambda: nn.init.trunc_normal_(table, std=.02))
            if tp_size > 1:
                table = table.chunk(tp_size, dim=-1)[tp_rank].contiguous()
            self.relative_position_bias_table = nn.Parameter(table)
            self.register_buffer("relative_position_index", relative_position_index(wh, ww))
            if factorized:
                self.relative_position_bias_table.terra_grad_reduce_group = TP_LABEL

        for k, name in enumerate(("q_linear", "k_linear", "v_linear"), start=1):
            if factorized:
                w, b = sharded_linear_tensors(embedding_dim, embedding_dim, tp_rank, tp_size, 0, True, seed(k))
                lin = linear_from_tensors(w, b)
                _tag(lin, TP_LABEL)
            else:
                lin = make_linear_with_seed(embedding_dim, embedding_dim, True, seed(k))
            setattr(self, name, lin)
        if factorized:
            w, b = sharded_linear_tensors(embedding_dim, embedding_dim, tp_rank, tp_size, -1, False, seed(4))
            self.proj = linear_from_tensors(w, None)
            _tag(self.proj, TP_LABEL)
            self.proj_bias = nn.Parameter(b)
        else:
            self.proj = make_linear_with_seed(embedding_dim, embedding_dim, True, seed(4))

    def bias_table(self) -> Optional[torch.Tensor]:
        """The table for differentiable code that reads it in fp32 (see ``ops/packed.py::fp32_param``)."""
        return fp32_param(self.relative_position_bias_table) if self.use_relative_position_bias else None


class SwinAttentionHalf(nn.Module):
    """norm1 + window attention + shortcut; odd layers are the shifted-window ones."""

    def __init__(self, layer_idx, embedding_dim, window_size, num_heads, use_attn_mask=True,
                 use_relative_position_bias=True, init_seed_base=None, pctx=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.pctx = pctx
        self.shifted = (layer_idx % 2 == 1)
        self.window_size = to_2tuple(window_size)
        self.use_attn_mask = use_attn_mask
        self.norm1 = nn.LayerNorm(embedding_dim)
        seed = None if init_seed_base is None else int(init_seed_base) + int(layer_idx) * 100
        factorized = pctx is not None and (pctx.sp > 1 or pctx.tp > 1)
        self.attn = WindowAttention(embedding_dim, self.window_size, num_heads, use_relative_position_bias, seed,
                                    factorized, pctx.tp if pctx is not None else 1, pctx.tp_rank if pctx is not None else 0)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        # checkpoints written by the reference carry a materialised shift mask; it is derived in-kernel here
        state_dict.pop(prefix + "attn_mask", None)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def forward(self, x):
        return self.pctx.attention_half(x, self)


class MlpHalf(nn.Module):
    """norm2 + fc1 + GELU + fc2 + shortcut."""

    def __init__(self, in_features, hidden_features, init_seed_base=None, pctx=None):
        super().__init__()
        self.pctx = pctx
        self.norm2 = nn.LayerNorm(in_features)
        s1 = None if init_seed_base is None else init_seed_base + 1
        s2 = None if init_seed_base is None else init_seed_base + 2
        self.tp = pctx.tp if pctx is not None else 1
        if self.tp > 1:
            w1, b1 = sharded_linear_tensors(in_features, hidden_features, pctx.tp_rank, self.tp, 0, True, s1)
            w2, b2 = sharded_linear_tensors(hidden_features, in_features, pctx.tp_rank, self.tp, -1, False, s2)
            self.linear1 = linear_from_tensors(w1, b1)
            self.linear2 = linear_from_tensors(w2, None)
            _tag(self.linear1, TP_LABEL)
            _tag(self.linear2, TP_LABEL)
            self.bias2 = nn.Parameter(b2)
        else:
            self.fc1 = make_linear_with_seed(in_features, hidden_features, True, s1)
            self.fc2 = make_linear_with_seed(hidden_features, in_features, True, s2)

    def forward(self, x):
        return self.pctx.mlp_half(x, self)


class BasicLayer(nn.Module):
    """``depth`` x (attention half, MLP half), run segment by segment under the recompute scheduler."""

    def __init__(self, dim, input_resolution, depth, num_heads, window_size, pctx, recompute_config=None,
                 use_attn_mask=True, use_relative_position_bias=True, attention_init_seed_base=None,
                 mlp_init_seed_base=None, module_name="sequential_basic_layer"):
        super().__init__()
        heads = list(num_heads) if isinstance(num_heads, (list, tuple)) else [num_heads] * depth
        if len(heads) != depth:
            raise ValueError(f"per-layer num_heads needs {depth} entries, got {len(heads)}")
        self.blocks = nn.ModuleList([
            nn.Sequential(
                SwinAttentionHalf(i, dim, window_size, heads[i], use_attn_mask, use_relative_position_bias,
                                  attention_init_seed_base, pctx),
                MlpHalf(dim, dim * 4, None if mlp_init_seed_base is None else int(mlp_init_seed_base) + i * 100, pctx),
            ) for i in range(depth)
        ])
        self.use_checkpointing = "no"
        self.recompute_scheduler = SelectiveRecomputeScheduler(recompute_config, depth=depth,
                                                               input_resolution=input_resolution, hidden_dim=dim,
                                                               module_name=module_name)

    def run_blocks(self, start, end, x):
        for idx in range(start, end):
            x = self.blocks[idx](x)
        return x

    def forward(self, x):
        sched = self.recompute_scheduler
        if not sched.enabled:
            return self.run_blocks(0, len(self.blocks), x)
        for start, end, ckpt in sched.execution_segments():
            label = f"{sched.module_name}:{start}-{end}:{'checkpoint' if ckpt else 'plain'}"
            mark_memory_timeline("transformer_segment_pre", label)
            if ckpt:
                x = activation_checkpoint(lambda inp, s=start, e=end: self.run_blocks(s, e, inp), x,
                                          activation_config=dict(sched.config_for_block(start),
                                                                 offload=dict(sched.config_for_block(start).get("offload") or {},
                                                                              scope="transformer")))
            else:
                x = self.run_blocks(start, end, x)
            mark_memory_timeline("transformer_segment_post", label)
        return x


class CreditDownBlock(nn.Module):
    """3x3/s2 conv, then two (3x3 conv, GroupNorm, SiLU) with a shortcut (FuXi-style; models/utils.py:101-138)."""

    def __init__(self, in_chans, out_chans, num_groups, wrapped=False):
        super().__init__()
        self.conv = _conv(nn.Conv2d(in_chans, out_chans, kernel_size=3, stride=2, padding=1), wrapped)
        layers = []
        for _ in range(2):
            layers += [_conv(nn.Conv2d(out_chans, out_chans, kernel_size=3, stride=1, padding=1), wrapped),
                       nn.GroupNorm(num_groups, out_chans), nn.SiLU()]
        self.b = nn.Sequential(*layers)


class CreditUpBlock(nn.Module):
    """2x2/s2 transposed conv, then the same residual stack (models/utils.py:141-177)."""

    def __init__(self, in_chans, out_chans, num_groups, wrapped=False):
        super().__init__()
        self.conv = _conv(nn.ConvTranspose2d(in_chans, out_chans, kernel_size=2, stride=2), wrapped)
        layers = []
        for _ in range(2):
            layers += [_conv(nn.Conv2d(out_chans, out_chans, kernel_size=3, stride=1, padding=1), wrapped),
                       nn.GroupNorm(num_groups, out_chans), nn.SiLU()]
        self.b = nn.Sequential(*layers)


class _Wrapped(nn.Module):
    """The parallel build nests every convolution one level (``...conv.conv.weight``)."""

    def __init__(self, conv):
        super().__init__()
        self.conv = conv

    @property
    def weight(self):
        return self.conv.weight

    @property
    def bias(self):
        return self.conv.bias


def _conv(conv, wrapped):
    return _Wrapped(conv) if wrapped else conv


def unwrap(m):
    return m.conv if isinstance(m, _Wrapped) else m


class WrappedLinear(nn.Linear):
    """Marker subclass: patch embedding / recovery of the parallel build act on already patchified input."""
