"""Shared set-up of the four entry points: distributed bootstrap, config defaults, topology, model, optimizer, data
(what the reference repeats at the top of each script: train_scripts/train.py:40-53, 372-470; finetune.py:334-470;
test_pretrain.py:100-390; test_finetune.py:100-360)."""
from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from terra_b200 import global_env_config as G  # noqa: E402
from terra_b200.config import get_model_archi_params_and_other_params, load_yaml  # noqa: E402
from terra_b200.data.dataloader_utils import (get_dataloader_for_task, get_finetune_dataloader_for_task,  # noqa: E402
                                              resolve_required_tensors_from_dataloader,
                                              resolve_required_tensors_online_split_for_parallel)
from terra_b200.data.task_specific_data import get_task_specific_data  # noqa: E402
from terra_b200.distributed import init_distributed, set_random_seed  # noqa: E402
from terra_b200.models.get_model import get_model_for_train  # noqa: E402
from terra_b200.parallel.rank_manager import ParallelManager, SingleProcessManager  # noqa: E402
from terra_b200.utils.misc import count_parameters, dtype_from_precision, get_criterion  # noqa: E402

PRETRAIN_DEFAULTS = {
    "description": "terra_run", "train_path": "./outputs", "ckpt_start": False, "ckpt_epoch": 0, "start_epoch": 0,
    "num_pre_train_epochs": 1, "save_interval_epochs": 1, "max_train_steps_per_epoch": None, "precision": "bf16",
    "half_model": False, "clip_grad": False, "learning_rate": 1e-4, "warmup_steps": 100, "loss_func": "L1",
    "micro_batch_size": 1, "kaiming_init": True, "optimizer_config": 4, "use_splited_data": True,
    "use_fake_input": False, "fake_input_random": True, "fake_input_seed": 1234, "num_workers": 1,
}
FINETUNE_DEFAULTS = dict(PRETRAIN_DEFAULTS, num_finetune_epochs=1, finetune_lead_time=2, finetune_loss_reduction="mean",
                         save_interval_steps=0, ckpt_step=None, trained_model_config_path=None,
                         trained_model_checkpoint_path=None, trained_model_epoch=None, load_pretrained_from_wp_rank0=True,
                         skip_pretrained_state_suffixes=["attn_mask"], input_double_buffer=True)


def set_default_config(cfg: dict, defaults: dict) -> dict:
    for k, v in defaults.items():
        cfg.setdefault(k, v)
    if os.environ.get("TERRA_USE_FAKE_INPUT", "0") == "1":
        cfg["use_fake_input"] = True
    return cfg


def base_parser(description: str) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--data_parallel_group_size", type=int, default=1)
    ap.add_argument("--model_cfg", type=str, required=True)
    return ap


class Session:
    """Everything an entry point needs, built from a YAML path and the DP size."""

    def __init__(self, model_cfg_path: str, data_parallel_group_size: int, defaults: dict, backend=None):
        self.rank, self.world, self.device = init_distributed(backend)
        set_random_seed(1234)
        self.cfg = set_default_config(load_yaml(model_cfg_path), defaults)
        self.task_type = self.cfg.get("task_type", "glorys")
        self.model_type = self.cfg["model_type"]
        self.dp = data_parallel_group_size
        self.archi, self.other = get_model_archi_params_and_other_params(self.task_type, self.cfg, self.dp, self.world)
        o = self.other
        if self.world > 1:
            self.manager = ParallelManager(dp_size=self.dp, mp_size=o["mp_size"], wp_topo=o["wp_topo"],
                                           xfmr_wp_topo=o["xfmr_wp_topo"], rank=self.rank, world_size=self.world,
                                           device=self.device, window_assignment_mode=o["window_assignment_mode"],
                                           xfmr_sp_size=o["xfmr_sp_size"], tensor_parallel_size=o["tensor_parallel_size"],
                                           sp_tp_placement=o["sp_tp_placement"])
        else:
            self.manager = SingleProcessManager(self.device, o["window_assignment_mode"])
        self.model, self.engine, self.optimizer, self.gscaler, self.opt_state = get_model_for_train(
            self.archi, self.cfg, self.task_type, self.model_type, o["embedding_parallel_type"], o["attn_parallel_type"],
            o["mlp_parallel_type"], self.manager, self.device, self.cfg.get("kaiming_init", True))
        from terra_b200 import global_env_config as G

        if G.DEBUG_GRAD_HOOK and self.device.type != "cuda":
            # (on CUDA the fused kernels accumulate into the flat gradient arena without autograd leaf gradients;
            # there the step itself prints the arena's per-parameter sums after the backward pass)
            from terra_b200.runtime.grad_debug import install_grad_hooks

            self.grad_hooks = install_grad_hooks(self.model)
        self.precision = self.cfg["precision"]
        self.my_dtype = dtype_from_precision(self.precision)
        self.criterion = get_criterion(self.cfg["loss_func"])
        self.loss_fn = self.cfg["loss_func"] if self.device.type == "cuda" else self.criterion
        self.task_data = get_task_specific_data(self.task_type, self.device, self.opt_state, self.archi, self.other,
                                                self.manager, self.cfg["micro_batch_size"], self.model_type, self.cfg)
        self.data_dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        from terra_b200.runtime.watchdog import make_step_guard

        # failure detection between steps: peer heartbeats, the kernels' status word, stream-wait watchdogs
        self.guard = make_step_guard(self.device, self.rank, self.world, self.model, self.optimizer)

    def pretrain_loader(self, status=0):
        c = self.cfg
        return get_dataloader_for_task(self.task_type, c["micro_batch_size"], c["use_splited_data"], status,
                                       c.get("num_workers", c.get("dataloader_num_workers", 1)), manager=self.manager,
                                       model_type=self.model_type, model_archi_params=self.archi, other_params=self.other,
                                       use_fake_input=c["use_fake_input"], fake_input_random=c.get("fake_input_random", True),
                                       fake_input_seed=c.get("fake_input_seed", 1234), fake_length=int(c.get("fake_length", 64)))

    def finetune_loader(self, lead_time, status=0):
        c = self.cfg
        return get_finetune_dataloader_for_task(self.task_type, c["micro_batch_size"], lead_time, c["use_splited_data"],
                                                status, c.get("num_workers", c.get("dataloader_num_workers", 1)),
                                                manager=self.manager, model_type=self.model_type,
                                                model_archi_params=self.archi, other_params=self.other,
                                                use_fake_input=c["use_fake_input"],
                                                fake_input_random=c.get("fake_input_random", True),
                                                fake_input_seed=c.get("fake_input_seed", 1234),
                                                fake_length=int(c.get("fake_length", 64)),
                                                pin_memory=c.get("dataloader_pin_memory", True))

    def to_required_tensors(self, batch):
        if self.model_type in ("parallel", "hybrid") and not self.cfg["use_splited_data"]:
            return resolve_required_tensors_online_split_for_parallel(batch, self.device, self.data_dtype, self.archi,
                                                                      self.other, self.manager)
        return resolve_required_tensors_from_dataloader(batch, self.device, self.data_dtype, self.model_type,
                                                        self.archi["num_channels"])

    def is_log_rank(self) -> bool:
        return self.rank == 0

    def close(self):
        import torch.distributed as dist

        self.guard.close()

        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
