"""Model assembly.

``credit_hierarchical_swin``: patch embedding -> FuXi-style conv down block (x2) -> one Swin stage -> transposed-conv
up block (x2) -> patch recovery -> + input.  ``swin_reference``: the same without the sampling blocks.
Each exists as a *sequential* build (takes the raw NHWC field, pads and patchifies it itself; the CPU fp32 oracle)
and a *parallel* build (takes this rank's row stripe of the padded, patchified field ``[B, h_loc, w, p*p*C]``).
Parameter names and shapes follow the reference so that its checkpoints load
(models/reference_model/sequential_hierarchical_swin.py:25-449, parallel_hierarchical_swin.py:55-683).

Internally all activations are NHWC (conv stage) or window-major rows (transformer stage); on CUDA they are bf16
and every operator is an sm_100a kernel from ``terra_b200.ops``.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..global_env_config import ON_H200
from ..memory.activation import activation_checkpoint, activation_config_for_sampling
from ..ops import blocks as B
from ..ops.conv import conv3x3, conv_transpose2x2, groupnorm_silu
from ..parallel.context import ParallelContext
from ..profiler.memory_timeline import mark_memory_timeline
from ..utils.padding import get_padded_shape
from .init_utils import REFERENCE_INIT_SEEDS, make_with_seed
from .layers import BasicLayer, CreditDownBlock, CreditUpBlock, WrappedLinear, to_2tuple, unwrap


def patchify(x, p):
    """[B, H, W, C] -> [B, H/p, W/p, p*p*C] with (p1, p2, c) feature order."""
    Bn, H, W, C = x.shape
    return x.reshape(Bn, H // p, p, W // p, p, C).permute(0, 1, 3, 2, 4, 5).reshape(Bn, H // p, W // p, p * p * C)


def unpatchify(x, p):
    Bn, h, w, F = x.shape
    C = F // (p * p)
    return x.reshape(Bn, h, w, p, p, C).permute(0, 1, 3, 2, 4, 5).reshape(Bn, h * p, w * p, C)


class _SwinBase(nn.Module):
    """Shared forward machinery; subclasses define how parameters are named and what the input looks like."""

    has_sampling = True

    def _setup(self, *, height, width, num_channels, patch_size, window_size, embedding_dim, num_heads, num_layers,
               padding_scale, padding_spec, recompute_config, manager, use_attn_mask, use_relative_position_bias,
               parallel, window_assignment_mode="regular", depths=None):
        self.manager = manager
        self.patch_size = patch_size
        self.window_size = to_2tuple(window_size)
        self.embedding_dim = embedding_dim
        self.num_channels = num_channels
        self.parallel = parallel
        resolved = padding_spec.get("padded_shape") if padding_spec else None
        self.need_padding, self.initial_padding, self.padded_shape = get_padded_shape(
            height, width, patch_size, self.window_size, padding_scale=padding_scale, padded_shape=resolved,
            downsample=2 if self.has_sampling else 1)
        hp, wp = self.padded_shape[0] // patch_size, self.padded_shape[1] // patch_size
        self.patches_resolution = [hp, wp]
        self._param_sharder = None          # set by terra_b200.parallel.param_sharding when parameters are sharded
        ds = 2 if self.has_sampling else 1
        self.div_val = patch_size * ds
        self.token_hw = (hp // ds, wp // ds)
        if depths is not None:
            heads = []
            hl = list(num_heads) if isinstance(num_heads, (list, tuple)) else [num_heads] * len(depths)
            for d, h in zip(depths, hl):
                heads += [h] * d
            num_layers, num_heads = len(heads), heads
        self.num_layers = num_layers
        self.pctx = ParallelContext(manager if parallel else None, self.window_size, self.token_hw,
                                    window_assignment_mode=window_assignment_mode)
        self.recompute_config = recompute_config or {}
        self.layers = make_with_seed(
            REFERENCE_INIT_SEEDS["layers"],
            lambda: BasicLayer(embedding_dim, self.token_hw, num_layers, num_heads, self.window_size, self.pctx,
                               recompute_config, use_attn_mask, use_relative_position_bias,
                               REFERENCE_INIT_SEEDS["attention"], REFERENCE_INIT_SEEDS["mlp"],
                               "parallel_basic_layer" if parallel else "sequential_basic_layer"))
        self.recompute_scheduler = self.layers.recompute_scheduler
        self.down_recompute_config = dict(activation_config_for_sampling(self.recompute_config, "down"))
        self.up_recompute_config = dict(activation_config_for_sampling(self.recompute_config, "up"))
        for cfg in (self.down_recompute_config, self.up_recompute_config):
            cfg["offload"] = dict(cfg.get("offload") or {}, scope="sampling")
        enabled = bool(self.recompute_config.get("enabled", False))
        self.checkpoint_down_mode = str(self.recompute_config.get("checkpoint_down_mode", "none")) if enabled else "none"
        self.checkpoint_up_mode = str(self.recompute_config.get("checkpoint_up_mode", "none")) if enabled else "none"
        if self.checkpoint_down_mode.lower() != "none":
            self.checkpoint_down_mode = self.checkpoint_down_mode.upper()
        if self.checkpoint_up_mode.lower() != "none":
            self.checkpoint_up_mode = self.checkpoint_up_mode.upper()
        self.checkpoint_patch_embed = bool(self.recompute_config.get("checkpoint_patch_embed", False)) and enabled
        self.checkpoint_patch_recovery = bool(self.recompute_config.get("checkpoint_patch_recovery", False)) and enabled

    # ------------------------------------------------------------------ pieces (NHWC in, NHWC out)
    def _embed_linear(self):
        return self.patch_embed if isinstance(self.patch_embed, nn.Linear) else self.patch_embed.linear

    def _recovery_linear(self):
        return self.patch_recovery if isinstance(self.patch_recovery, nn.Linear) else self.patch_recovery.linear

    def _dom(self):
        return self.pctx.dom if self.parallel else None

    def _in_unit(self, mod, fn, *args):
        """Run a piece of the sampling path with the parameters of ``mod`` present: a plain call, unless the parameters
        are sharded with the sampling modules as units of their own (``terra_b200.parallel.param_sharding``)."""
        sharder = getattr(self, "_param_sharder", None)
        if sharder is None:
            return fn(*args)
        return sharder.run_in_unit(mod, fn, *args)

    def _patch_embed(self, patches):
        def run(patches):
            Bn, h, w, F = patches.shape
            y = B.linear(patches.reshape(-1, F), self._embed_linear(), need_dx=patches.requires_grad)
            return y.reshape(Bn, h, w, -1)
        return self._in_unit(self.patch_embed, run, patches)

    def _down_conv(self, x):
        return self._in_unit(self.down_blk, lambda t: conv3x3(t, unwrap(self.down_blk.conv), 2, self._dom()), x)

    def _up_conv(self, x):
        return self._in_unit(self.up_blk, lambda t: conv_transpose2x2(t, unwrap(self.up_blk.conv)), x)

    def _residual_first(self, blk, x):
        return self._in_unit(blk, lambda t: groupnorm_silu(conv3x3(t, unwrap(blk.b[0]), 1, self._dom()), blk.b[1], None,
                                                           self._dom()), x)

    def _residual_second(self, blk, x, shortcut):
        return self._in_unit(blk, lambda t, s: groupnorm_silu(conv3x3(t, unwrap(blk.b[3]), 1, self._dom()), blk.b[4], s,
                                                              self._dom()), x, shortcut)

    def _down_block(self, x):
        def run(x):
            x = self._down_conv(x)
            return self._residual_second(self.down_blk, self._residual_first(self.down_blk, x), x)
        return self._in_unit(self.down_blk, run, x)

    def _up_block(self, x):
        def run(x):
            x = self._up_conv(x)
            return self._residual_second(self.up_blk, self._residual_first(self.up_blk, x), x)
        return self._in_unit(self.up_blk, run, x)

    def _patch_recovery(self, x, residual=None):
        def run(x, residual):
            Bn, h, w, D = x.shape
            res = None if residual is None else residual.reshape(Bn * h * w, -1)
            y = B.linear(x.reshape(-1, D), self._recovery_linear(), residual=res)
            return y.reshape(Bn, h, w, -1)
        return self._in_unit(self.patch_recovery, run, x, residual)

    def _ckpt(self, fn, *args, cfg):
        label = getattr(fn, "__name__", "piece")
        mark_memory_timeline("checkpoint_edge_pre", label)
        out = activation_checkpoint(fn, *args, activation_config=cfg)
        mark_memory_timeline("checkpoint_edge_post", label)
        return out

    def _run_patch_embed_down(self, patches):
        mode = self.checkpoint_down_mode if self.has_sampling else "none"
        cfg = self.down_recompute_config
        mark_memory_timeline("sampling_down_enter", mode)
        if not self.has_sampling:
            out = self._ckpt(self._patch_embed, patches, cfg=cfg) if self.checkpoint_patch_embed else self._patch_embed(patches)
        elif mode == "D0":
            out = self._ckpt(lambda p: self._down_block(self._patch_embed(p)), patches, cfg=cfg)
        elif mode == "D1":
            x = self._ckpt(lambda p: self._down_conv(self._patch_embed(p)), patches, cfg=cfg)
            h = self._ckpt(lambda t: self._residual_first(self.down_blk, t), x, cfg=cfg)
            out = self._ckpt(lambda t, s: self._residual_second(self.down_blk, t, s), h, x, cfg=cfg)
        elif mode == "none":
            out = self._down_block(self._patch_embed(patches))
        else:
            raise ValueError(f"Unsupported down sampling checkpoint mode: {mode}")
        mark_memory_timeline("sampling_down_exit", mode)
        return out

    def _run_up_patch_recovery(self, x, residual):
        mode = self.checkpoint_up_mode if self.has_sampling else "none"
        cfg = self.up_recompute_config
        mark_memory_timeline("sampling_up_enter", mode)
        if not self.has_sampling:
            if self.checkpoint_patch_recovery:
                out = self._ckpt(lambda t, r: self._patch_recovery(t, r), x, residual, cfg=cfg)
            else:
                out = self._patch_recovery(x, residual)
        elif mode == "U0":
            out = self._ckpt(lambda t, r: self._patch_recovery(self._up_block(t), r), x, residual, cfg=cfg)
        elif mode == "U1":
            u = self._ckpt(lambda t: self._up_conv(t), x, cfg=cfg)
            h = self._ckpt(lambda t: self._residual_first(self.up_blk, t), u, cfg=cfg)
            h = self._ckpt(lambda t, s: self._residual_second(self.up_blk, t, s), h, u, cfg=cfg)
            out = self._ckpt(lambda t, r: self._patch_recovery(t, r), h, residual, cfg=cfg)
        elif mode == "none":
            out = self._patch_recovery(self._up_block(x), residual)
        else:
            raise ValueError(f"Unsupported up sampling checkpoint mode: {mode}")
        mark_memory_timeline("sampling_up_exit", mode)
        return out

    def _core(self, patches, residual):
        """patches / residual: [B, h_loc, w, p*p*C] (residual may be None) -> same shape."""
        Bn = patches.shape[0]
        x = self._run_patch_embed_down(patches)
        rows = self.pctx.stripe_to_windows(x)
        rows = self.layers(rows)
        x = self.pctx.windows_to_stripe(rows, Bn)
        return self._run_up_patch_recovery(x, residual)

    def _compute_dtype(self, x):
        return torch.bfloat16 if x.is_cuda else torch.float32

    def _ensure_arena(self, x):
        if x.is_cuda and getattr(self, "_param_arena", None) is None:
            from ..utils.flat_params import ParamArena

            ParamArena(self)


class SequentialHierarchicalSwin(_SwinBase):
    def __init__(self, padding_scale, num_channels=93, kaiming_init=True, patch_size=6, window_size=6, height=720,
                 width=1440, embedding_dim=768, num_heads=-1, num_layers=2, recompute_config=None, manager=None,
                 use_attn_mask=True, use_relative_position_bias=True, use_flash_attention=False, padding_spec=None,
                 depths=None):
        super().__init__()
        self._setup(height=height, width=width, num_channels=num_channels, patch_size=patch_size,
                    window_size=window_size, embedding_dim=embedding_dim, num_heads=num_heads, num_layers=num_layers,
                    padding_scale=padding_scale, padding_spec=padding_spec, recompute_config=recompute_config,
                    manager=manager, use_attn_mask=use_attn_mask, use_relative_position_bias=use_relative_position_bias,
                    parallel=False, depths=depths)
        F = num_channels * patch_size * patch_size
        self.patch_embed = make_with_seed(REFERENCE_INIT_SEEDS["patch_embed"], lambda: _LinearHolder(F, embedding_dim))
        self.patch_recovery = make_with_seed(REFERENCE_INIT_SEEDS["patch_recovery"], lambda: _LinearHolder(embedding_dim, F))
        if self.has_sampling:
            self.down_blk = make_with_seed(REFERENCE_INIT_SEEDS["down_blk"],
                                           lambda: CreditDownBlock(embedding_dim, embedding_dim, 32))
            self.up_blk = make_with_seed(REFERENCE_INIT_SEEDS["up_blk"],
                                         lambda: CreditUpBlock(embedding_dim, embedding_dim, 32))
        self.input_nchw = ON_H200

    def forward(self, input):
        self._ensure_arena(input)
        x = input.permute(0, 2, 3, 1) if self.input_nchw else input
        raw_h, raw_w = x.shape[1], x.shape[2]
        xin = x.to(self._compute_dtype(x))
        if self.need_padding:
            left, right, top, bottom = self.initial_padding
            xin = torch.nn.functional.pad(xin, (0, 0, left, right, top, bottom))
        patches = patchify(xin, self.patch_size).contiguous()
        y = unpatchify(self._core(patches, None), self.patch_size)
        if self.need_padding:
            left, right, top, bottom = self.initial_padding
            y = y[:, top:top + raw_h, left:left + raw_w, :]
        y = y + x.to(y.dtype)
        return y.permute(0, 3, 1, 2).contiguous() if self.input_nchw else y


class SequentialSwinReference(SequentialHierarchicalSwin):
    has_sampling = False


class _LinearHolder(nn.Module):
    """The sequential build names its patch projections ``patch_embed.linear.*`` / ``patch_recovery.linear.*``."""

    def __init__(self, fin, fout):
        super().__init__()
        self.linear = nn.Linear(fin, fout, bias=True)


class ParallelHierarchicalSwin(_SwinBase):
    def __init__(self, height, width, num_channels, patch_size, embedding_dim, num_layers, num_heads, window_size,
                 kaiming_init=True, manager=None, device=None, padding_scale=4, embedding_parallel_type=None,
                 recompute_config=None, use_attn_mask=True, use_relative_position_bias=True, use_flash_attention=False,
                 padding_spec=None, depths=None):
        super().__init__()
        mode = getattr(manager, "window_assignment_mode", "regular") if manager is not None else "regular"
        self._setup(height=height, width=width, num_channels=num_channels, patch_size=patch_size,
                    window_size=window_size, embedding_dim=embedding_dim, num_heads=num_heads, num_layers=num_layers,
                    padding_scale=padding_scale, padding_spec=padding_spec, recompute_config=recompute_config,
                    manager=manager, use_attn_mask=use_attn_mask, use_relative_position_bias=use_relative_position_bias,
                    parallel=True, window_assignment_mode=mode, depths=depths)
        self.rank = manager.rank if manager is not None else 0
        self.wp_rank = manager.get_wp_rank() if manager is not None else 0
        self.wp_group_size = manager.get_wp_group_size() if manager is not None else 1
        if manager is not None:
            manager.update_window_info(self.pctx.nWh, self.pctx.nWw)
        F = num_channels * patch_size * patch_size
        self.patch_embed = make_with_seed(REFERENCE_INIT_SEEDS["patch_embed"], lambda: WrappedLinear(F, embedding_dim, bias=True))
        self.patch_recovery = make_with_seed(REFERENCE_INIT_SEEDS["patch_recovery"], lambda: WrappedLinear(embedding_dim, F, bias=True))
        if self.has_sampling:
            self.down_blk = make_with_seed(REFERENCE_INIT_SEEDS["down_blk"],
                                           lambda: CreditDownBlock(embedding_dim, embedding_dim, 32, wrapped=True))
            self.up_blk = make_with_seed(REFERENCE_INIT_SEEDS["up_blk"],
                                         lambda: CreditUpBlock(embedding_dim, embedding_dim, 32, wrapped=True))
        # every parameter is replicated over (part of) the window-parallel group: its gradient is summed there
        self.mp_all_reduce_list = []
        for name, p in self.named_parameters():
            p.allreduce_wp_group = True
            p.full_name = name
            self.mp_all_reduce_list.append(name)

    def forward(self, input):
        """input: ``[B, h_loc, w, p*p*C]`` row stripe of the padded, patchified field."""
        self._ensure_arena(input)
        x = input.to(self._compute_dtype(input)).contiguous()
        return self._core(x, x)


class ParallelSwinReference(ParallelHierarchicalSwin):
    has_sampling = False
