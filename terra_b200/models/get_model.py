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
    precision = model_config.get("precision", "bf16")
    if precision not in ("fp32", "fp16", "bf16"):
        raise ValueError(f"precision must be fp32, fp16 or bf16, got {precision!r}")
    model = get_model(model_archi_params, task_type, model_config.get("model_architecture"), kaiming_init, model_type,
                      embedding_parallel_type, attn_parallel_type, mlp_parallel_type, manager, device)
    ParamArena(model)
    state = optimizer_state_tuple(model_config.get("optimizer_config", 4), model_config.get("tensor_parallel_size", 1))
    optimizer = get_optimizer(model, model_config, manager, use_dist_opt=state[3])
    gscaler = None
    on_cuda = device is not None and torch.device(device).type == "cuda"
    if on_cuda and precision == "fp32":
        raise ValueError("precision: fp32 is not available on CUDA: the sm_100a kernels compute in bf16 with fp32 "
                         "accumulation, masters and optimizer state. Use precision: bf16 (or fp16 for loss scaling); "
                         "the fp32 model runs on the CPU build, which is the numerical oracle.")
    if precision == "fp16":
        if on_cuda:
            import warnings

            from ..optim.grad_scaler import LossScaler

            warnings.warn("precision: fp16 -> bf16 arithmetic (the kernels have no fp16 path) with the dynamic loss "
                          "scaler, inf/nan skip and fp16-only clipping kept", stacklevel=2)
            gscaler = LossScaler(init_scale=float(model_config.get("loss_scale_init", 65536.0)),
                                 growth_interval=int(model_config.get("loss_scale_growth_interval", 2000)))
        else:
            gscaler = torch.amp.GradScaler("cpu", enabled=False)
    oc = int(model_config.get("optimizer_config", 4))
    if oc in (1, 2, 3, 5, 7, 8, 9) and not getattr(get_model_for_train, "_warned_fallback", False):
        import warnings

        get_model_for_train._warned_fallback = True
        warnings.warn(f"optimizer_config {oc}: DeepSpeed / FSDP wrappers are not used; this framework runs its own "
                      "sharded optimizer (fp32 masters and moments sharded over the replica group, bf16 working copy "
                      "replicated)", stacklevel=2)
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
