"""Model / optimizer factory (reference: models/model_utils/get_model.py:987-1359).

``get_model_for_train`` returns ``(model, engine, optimizer, gscaler, (USE_DDP, USE_FSDP, ZERO_STAGE, USE_DIST_OPT))``.
``optimizer_config`` keeps its meaning as a selector of the parallel-optimizer stack, mapped onto what this
framework implements natively:

  4          replicated AdamW; gradients averaged over DP (and summed over WP / TP replicas) in one collective
             per parameter class - the role DDP + ``grad_post_process`` play in the reference
  6          ``DistributedAdamW``: reduce-scatter + sharded fp32 update + all-gather
  5, 7, 8, 9 the reference's FSDP configurations, and 3 (ZeRO stage 3): parameters, gradients and optimizer state
             sharded; a unit's parameters are all-gathered while it runs (``terra_b200.parallel.param_sharding``).
             5 shards the model as one unit; 7 (TP = 1) and 8 / 9 (TP > 1) shard per ``FSDP_WRAPPER_CFG`` transformer
             blocks, TP-sharded parameters over the ranks at the same TP rank, the others over the full replica group
  2          ZeRO stage 2: the same units with the parameters kept between a unit's forward and backward pass
             (gathered once per step, gradients and optimizer state sharded)
  1          ZeRO stage 1: the sharded-optimizer path of 6 (state and updates sharded, parameters replicated)
  0          replicated AdamW

``TERRA_PARAM_SHARDING=0`` runs 2 / 3 / 5 / 7 / 8 / 9 on the sharded-optimizer path instead (parameters replicated).
"""
from __future__ import annotations

import os

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


PARAM_SHARDING_CONFIGS = (2, 3, 5, 7, 8, 9)


def _sharded_parameters(model, archi, model_config, manager, oc):
    """Cut the model into parameter-sharding units and return their optimizer (reference:
    models/model_utils/get_model.py:1196-1283)."""
    import torch.distributed as dist

    from .. import global_env_config as G
    from ..optim.sharded_param_adamw import ShardedParamAdamW
    from ..parallel.param_sharding import ParamSharder

    live = dist.is_available() and dist.is_initialized()

    def resolve(label):
        if manager is None or not live:
            return None, 0, 1
        if label == "xfmr_tp_param_group":
            g = manager.xfmr_tp_param_replica_group
        elif label == "full":
            g = manager.full_param_replica_group
        else:
            raise ValueError(f"Unknown terra_grad_reduce_group: {label}")
        if g is None and dist.get_world_size() == 1:
            return None, 0, 1
        if g is None:
            raise ValueError(f"optimizer_config={oc} requires manager.{'xfmr_tp_param_replica_group' if label != 'full' else 'full_param_replica_group'}.")
        return g, dist.get_rank(g), dist.get_world_size(g)

    sharder = ParamSharder(model, resolve, blocks_per_unit=G.FSDP_WRAPPER_CFG, whole_model=(oc == 5),
                           prefetch=archi.get("FSDP_CONFIG7_PREFETCH_POLICY", "none"), reshard_after_forward=(oc != 2),
                           sampling_units=int(archi.get("FSDP_SAMPLING_WRAPPER_CFG", 0) or 0) > 0)
    if manager is None or manager.get_rank() == 0:
        print(f"[FSDP] optimizer_config={oc} {sharder.describe()}, wrapper_cfg={G.FSDP_WRAPPER_CFG}, "
              f"sampling_wrapper_cfg={int(archi.get('FSDP_SAMPLING_WRAPPER_CFG', 0) or 0)}", flush=True)
    if G.DEBUG_GRAD_HOOK and next(model.parameters()).is_cuda:
        # on CUDA the kernels write gradients in place and no autograd hook fires: report when a unit is left
        from ..runtime.grad_debug import report_unit_gradients

        sharder.observe_gradients(report_unit_gradients)
    opt = ShardedParamAdamW(sharder, lr=float(model_config.get("learning_rate", 1e-4)), betas=(0.9, 0.95), weight_decay=0.1,
                            manager=manager)
    opt.global_step = 0
    return opt


def get_model_for_train(model_archi_params, model_config, task_type="glorys", model_type="sequential",
                        embedding_parallel_type=None, attn_parallel_type=None, mlp_parallel_type=None, manager=None,
                        device=None, kaiming_init=True):
    precision = model_config.get("precision", "bf16")
    if precision not in ("fp32", "fp16", "bf16"):
        raise ValueError(f"precision must be fp32, fp16 or bf16, got {precision!r}")
    oc = int(model_config.get("optimizer_config", 4))
    tp = int(model_config.get("tensor_parallel_size", 1) or 1)
    if oc in (5, 7) and tp > 1:
        raise ValueError(f"optimizer_config={oc} (FSDP) is currently only allowed when tensor_parallel_size == 1. Got "
                         f"tensor_parallel_size={tp}. Use optimizer_config=8/9 for TP-aware FSDP or optimizer_config=6 "
                         "for the custom distributed optimizer.")
    if oc in (8, 9) and tp <= 1:
        raise ValueError(f"optimizer_config={oc} (TP-aware FSDP) requires tensor_parallel_size > 1. Got "
                         f"tensor_parallel_size={tp}. Use optimizer_config=7 for block-level FSDP.")
    model = get_model(model_archi_params, task_type, model_config.get("model_architecture"), kaiming_init, model_type,
                      embedding_parallel_type, attn_parallel_type, mlp_parallel_type, manager, device)
    state = optimizer_state_tuple(oc, tp)
    shard_params = oc in PARAM_SHARDING_CONFIGS and os.environ.get("TERRA_PARAM_SHARDING", "1") != "0"
    if shard_params:
        optimizer = _sharded_parameters(model, model_archi_params, model_config, manager, oc)
    else:
        ParamArena(model)
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
    if oc == 1 or (oc in PARAM_SHARDING_CONFIGS and not shard_params):
        if not getattr(get_model_for_train, "_warned_fallback", False):
            import warnings

            get_model_for_train._warned_fallback = True
            warnings.warn(f"optimizer_config {oc}: runs on the sharded optimizer (fp32 masters' updates and moments "
                          "sharded over the replica group, gradients reduce-scattered, parameters replicated)",
                          stacklevel=2)
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
