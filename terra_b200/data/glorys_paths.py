"""Where the GLORYS tensors live (environment contract of the reference: dataloader/glorys_paths.py:21-85)."""
from __future__ import annotations

import os
from typing import Iterable, Optional


def _first_existing(candidates: Iterable[Optional[str]], kind: str, description: str) -> str:
    tried = []
    for c in candidates:
        if not c:
            continue
        tried.append(c)
        if (kind == "dir" and os.path.isdir(c)) or (kind == "file" and os.path.isfile(c)):
            return c
    raise FileNotFoundError(f"{description} not found; tried: {tried or 'nothing (set the TERRA_GLORYS_* variables)'}")


def resolve_glorys_sequential_root(norm_type="zs", data_precision="fp16", explicit_root=None) -> str:
    env = os.environ.get("TERRA_GLORYS_MM_ROOT" if norm_type == "mm" else "TERRA_GLORYS_ZS_ROOT")
    return _first_existing([explicit_root, env, os.environ.get("TERRA_GLORYS_SEQUENTIAL_ROOT")], "dir",
                           f"GLORYS sequential data ({norm_type}, {data_precision})")


def resolve_glorys_parallel_root(explicit_root=None) -> str:
    return _first_existing([explicit_root, os.environ.get("TERRA_GLORYS_PARALLEL_ROOT")], "dir", "GLORYS pre-split data")


def get_glorys_parallel_file_path_prefix(embedding_parallel_type, height, width, wp_topo, patch_size, window_size,
                                         padding_scale, norm_type="zs", data_precision="fp16", padding_spec=None,
                                         explicit_root=None) -> str:
    """Directory of the pre-split tensors of one layout: ``<root>/<layout tag>/`` with ``wp_rank_{r}`` below it."""
    root = resolve_glorys_parallel_root(explicit_root)
    padded = tuple(padding_spec["padded_shape"]) if padding_spec else None
    tag = (f"{embedding_parallel_type}_h{height}_w{width}_wp{wp_topo[0]}x{wp_topo[1]}_p{patch_size}_ws{window_size}"
           f"_{'pad%dx%d' % padded if padded else 'ps%s' % padding_scale}_{norm_type}_{data_precision}")
    return os.path.join(root, tag)


def resolve_glorys_mask_path(explicit_path=None) -> str:
    return _first_existing([explicit_path, os.environ.get("TERRA_GLORYS_MASK_PATH")], "file", "GLORYS land-sea mask")
