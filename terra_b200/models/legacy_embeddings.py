"""The reference's older embedding variants (models/patch_embedding.py:103-378): patch embedding / recovery as a plain
linear over this rank's windows (``embedding_parallel_type: window_embedding``), or as a 2-D distributed GEMM over
a model-parallel group with the weight sharded by rows or by columns (``domain_parallel`` / ``window_domain``).

No shipped configuration selects them (the default is ``window_linear``, i.e. ``WrappedLinear`` on row stripes); they
are kept so that a model description written against those names still builds. The distributed form runs on
``parallel/dist_matmul.py``; its process group is passed in directly (``manager.model_parallel_group`` in the
reference).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import global_env_config as G
from ..parallel import collectives as C
from ..parallel.dist_matmul import LAYOUTS, shard, xwt_apply


def split_embedding_weight_and_bias(linear_in_dim: int, linear_out_dim: int, rank: int, group_size: int, input_split: str,
                                    output_split: str, use_bias: bool = True) -> Tuple[nn.Parameter, Optional[nn.Parameter]]:
    """This rank's shard of a freshly initialised ``nn.Linear(linear_in_dim, linear_out_dim)`` (every rank draws the same
    full matrix from the current RNG state, as the reference does, and keeps its part): the columns
    ``[rank * in / n, ...)`` when the activation is cut by columns, the rows ``[rank * out / n, ...)`` when it is cut
    by rows; the bias whole for row-sharded outputs and cut like the output columns otherwise."""
    if input_split not in LAYOUTS or output_split not in LAYOUTS:
        raise ValueError(f"unrecognized split {input_split!r} -> {output_split!r}")
    full = nn.Linear(linear_in_dim, linear_out_dim, bias=use_bias)
    w = shard(full.weight.detach(), "(1,n)" if input_split == "(1,n)" else "(m,1)", rank, group_size).clone()
    b = None
    if use_bias:
        b = full.bias.detach()
        if output_split == "(1,n)":
            b = shard(b[None], "(1,n)", rank, group_size)[0]
        b = nn.Parameter(b.clone())
    return nn.Parameter(w), b


class _DomainParaLinear(nn.Module):
    def __init__(self, fin: int, fout: int, group, input_split: str, output_split: str, split_param: bool):
        super().__init__()
        self.group, self.input_split, self.output_split, self.split_param = group, input_split, output_split, split_param
        if split_param:
            self.weight, self.bias = split_embedding_weight_and_bias(fin, fout, C.group_rank(group), C.group_size(group),
                                                                     input_split, output_split)
        elif (input_split, output_split) == ("(m,1)", "(m,1)"):
            self.linear = nn.Linear(fin, fout)           # replicated weight, rows stay where they are
        else:
            raise ValueError("an unsplit weight is only supported for '(m,1)' -> '(m,1)'")

    def forward(self, x):
        if not self.split_param:
            return self.linear(x)
        return xwt_apply(x, self.weight, self.bias, self.group, self.input_split, self.output_split)


class DomainParaPatchEmbedding(_DomainParaLinear):
    """``[..., patch^2 * channels] -> [..., embedding_dim]`` over a model-parallel group
    (models/patch_embedding.py:206-262)."""

    def __init__(self, group=None, patch_size: int = -1, num_channel: int = -1, embedding_dim: int = -1,
                 input_split: Optional[str] = None, output_split: Optional[str] = None, split_param: Optional[bool] = None):
        super().__init__(num_channel * patch_size * patch_size, embedding_dim, group,
                         input_split or G.EMB_1_input_split, output_split or G.EMB_1_output_split,
                         G.EMB_1_SPLIT_PARAM if split_param is None else split_param)


class DomainParaPatchRecovery(_DomainParaLinear):
    """``[..., embedding_dim] -> [..., patch^2 * channels]`` (models/patch_embedding.py:264-324)."""

    def __init__(self, group=None, patch_size: int = -1, num_channel: int = -1, embedding_dim: int = -1,
                 input_split: Optional[str] = None, output_split: Optional[str] = None, split_param: Optional[bool] = None):
        super().__init__(embedding_dim, num_channel * patch_size * patch_size, group,
                         input_split or G.EMB_2_input_split, output_split or G.EMB_2_output_split,
                         G.EMB_2_SPLIT_PARAM if split_param is None else split_param)


class WindowParaPatchEmbedding(nn.Module):
    """A linear over the patches of this rank's windows, ``[B, windows, tokens, patch^2 * channels]`` in
    (models/patch_embedding.py:327-352)."""

    def __init__(self, patch_size: int = -1, num_channel: int = -1, embedding_dim: int = -1):
        super().__init__()
        self.embedding_dim = embedding_dim
        self.linear = nn.Linear(num_channel * patch_size * patch_size, embedding_dim)

    def forward(self, x):
        return self.linear(x)


class WindowParaPatchRecovery(nn.Module):
    """The inverse projection on window-major activations (models/patch_embedding.py:355-377)."""

    def __init__(self, patch_size: int = -1, num_channel: int = -1, embedding_dim: int = -1):
        super().__init__()
        self.linear = nn.Linear(embedding_dim, num_channel * patch_size * patch_size)

    def forward(self, x):
        return self.linear(x)
