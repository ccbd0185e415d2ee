"""Model / optimizer factory (reference: models/model_utils/get_model.py:987-1359).

``get_model_for_train`` returns ``(model, engine, optimizer, gscaler, (USE_DDP, USE_FSDP, ZERO_STAGE, USE_DIST_OPT))``.
``optimizer_config`` keeps its meaning as a selector of the parallel-optimizer stack, mapped onto what this
framework implements natively:

  4          replicated AdamW; gradients averaged over DP (and summed over WP / TP replicas) in one collective
             per parameter class - the role DDP + ``grad_post_process`` play in the reference
  6          ``DistributedAdamW``: reduce-scatter + sharded fp32 update + all-gather
  1, 2, 3    ZeRO stages, 5 / 7 / 8 / 9 FSDP variants: run on the same sharded-optimizer path as 6 (optimizer state
             and master weights sharded; parameters stay replicated in bf16 - 2 bytes per parameter - instead of
             being re-gathered per unit)
  0          replicated AdamW
"""
from __future__ import annotations

import torch

from ..optim.utils import get_optimizer
from ..utils.flat_params import ParamArena
from .hierarchical_swin import (ParallelHierarchicalSwin, ParallelSwinReference, SequentialHierarchicalSwin,
                                SequentialSwinReference)

_FAMILIES = {
    "credit_hierarchical_swin": (SequentialHierarchicalSwin, ParallelHierarchicalSwin),
    "swin_reference": (SequentialSwinReference, ParallelSwinReference),
}


def get_model(model_archi_params, task_type="glorys", model_architecture=None, kaiming_init=True,
              model_type="sequential", embedding_parallel_type=None, attn_parallel_type=None, mlp_parallel_type=None,
              manager=None, device=None):
    arch = model_architecture or model_archi_params.get("model_architecture")
    if arch not in _FAMILIES:
        raise ValueError(f"Unsupported model_architecture: {arch}")
    seq_cls, par_cls = _FAMILIES[arch]
    p = model_archi_params
    common = dict(num_channels=p["num_channels"], patch_size=p["patch_size"], window_size=p["window_size"],
                  height=p["height"], width=p["width"], embedding_dim=p["embedding_dim"], num_heads=p["num_heads"],
                  num_layers=p["num_layers"], recompute_config=p.get("activation"), manager=manager,
                  use_attn_mask=p.get("use_attn_mask", True),
                  use_relative_position_bias=p.get("use_relative_position_bias", True),
                  use_flash_attention=p.get("USE_FLASH_ATTENTION", False), padding_spec=p.get("padding_spec"),
                  padding_scale=p.get("padding_scale", 1), kaiming_init=kaiming_init, depths=p.get("depths"))
    if model_type == "sequential":
        model = seq_cls(**common)
    elif model_type in ("parallel", "hybrid"):
        model = par_cls(device=device, embedding_parallel_type=embedding_parallel_type, **common)
    else:
        raise ValueError(f"unrecognized model_type {model_type}")
    if device is not None:
        model = model.to(device)
    return model


def optimizer_state_tuple(optimizer_config: int, tensor_parallel_size: int = 1):
    oc = int(optimizer_config)
    if oc not in range(0, 10):
        raise ValueError(f"optimizer_config must be in 0..9, got {oc}")
    use_dist = oc in (1, 2, 3, 5, 6, 7, 8, 9)
    use_ddp = oc == 4
    zero_stage = oc if oc in (0, 1, 2, 3) else -1
    # FSDP averages the loss over DP x WP itself in the reference; the sharded optimizer here reduces
    # gradients like config 6, so the non-FSDP loss convention applies to every value.
    return use_ddp, False, zero_stage, use_dist


def get_model_for_train(model_archi_params, model_config, task_type="glorys", model_type="sequential",
                        embedding_parallel_type=None, attn_parallel_type=None, mlp_parallel_type=None, manager=None,
                        device=None, kaiming_init=True):
    model = get_model(model_archi_params, task_type, model_config.get("model_architecture"), kaiming_init, model_type,
                      embedding_parallel_type, attn_parallel_type, mlp_parallel_type, manager, device)
    ParamArena(model)
    state = optimizer_state_tuple(model_config.get("optimizer_config", 4), model_config.get("tensor_parallel_size", 1))
    optimizer = get_optimizer(model, model_config, manager, use_dist_opt=state[3])
    gscaler = None
    if model_config.get("precision", "bf16") == "fp16" and not (device is not None and torch.device(device).type == "cuda"):
        gscaler = torch.amp.GradScaler("cpu", enabled=False)
    on_cuda = device is not None and torch.device(device).type == "cuda"
    if on_cuda and manager is not None and manager.wp_size > 1 and model_config.get("comm_backend", "nvlink") == "nvlink":
        from ..parallel import nvlink

        nvlink.attach(model, optimizer, manager)
    return model, None, optimizer, gscaler, state


def load_model_ckpt(model, path, map_location="cpu"):
    """Legacy evaluation loader: a file holding ``model_state_dict`` (or the bare state dict)."""
    blob = torch.load(path, map_location=map_location)
    sd = blob.get("model_state_dict", blob) if isinstance(blob, dict) else blob
    sd = {(k[len("module."):] if k.startswith("module.") else k): v for k, v in sd.items()}
    model.load_state_dict(sd, strict=False)
    return model
