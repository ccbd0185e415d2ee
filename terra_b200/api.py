"""Public training API: ``Trainer(config)`` builds topology, model, optimizer and the input pipeline;
``trainer.step(batch)`` runs one optimisation step on a batch that lives in pinned host memory and returns the
loss as a Python float.

    trainer = Trainer("configs/model/pretrain/x.yaml", data_parallel_group_size=1)
    batch = trainer.synthetic_batch(sample=0)           # pinned host tensors of this rank's stripe
    loss = trainer.step(batch)
    trainer.save_checkpoint(epoch=0, loss=loss)         # and trainer.load_checkpoint(epoch=0) to resume

The same object backs ``train_scripts/train.py`` and ``bench.py``.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Union

import torch
import torch.distributed as dist

from . import _ext
from .config import get_model_archi_params_and_other_params, load_yaml
from .data.synthetic import land_mask_for_rank, synthetic_batch
from .distributed import init_distributed, set_random_seed
from .models.get_model import get_model_for_train
from .parallel.rank_manager import ParallelManager, SingleProcessManager
from .runtime.run_model import one_step_train_production


class Trainer:
    def __init__(self, model_config: Union[str, dict], data_parallel_group_size: int = 1, backend: Optional[str] = None,
                 seed: int = 1234):
        cfg = load_yaml(model_config) if isinstance(model_config, str) else dict(model_config)
        self.cfg = cfg
        self.rank, self.world, self.device = init_distributed(backend)
        set_random_seed(seed)
        self.task_type = cfg.get("task_type", "glorys")
        self.model_type = cfg["model_type"]
        self.archi, self.other = get_model_archi_params_and_other_params(self.task_type, cfg, data_parallel_group_size, self.world)
        if self.world > 1:
            self.manager = ParallelManager(
                dp_size=data_parallel_group_size, mp_size=self.other["mp_size"], wp_topo=self.other["wp_topo"],
                xfmr_wp_topo=self.other["xfmr_wp_topo"], rank=self.rank, world_size=self.world, device=self.device,
                window_assignment_mode=self.other["window_assignment_mode"], xfmr_sp_size=self.other["xfmr_sp_size"],
                tensor_parallel_size=self.other["tensor_parallel_size"], sp_tp_placement=self.other["sp_tp_placement"])
        else:
            self.manager = SingleProcessManager(self.device, self.other["window_assignment_mode"])
        self.model, self.engine, self.optimizer, self.gscaler, self.opt_state = get_model_for_train(
            self.archi, cfg, self.task_type, self.model_type, self.other["embedding_parallel_type"],
            self.other["attn_parallel_type"], self.other["mlp_parallel_type"], self.manager, self.device)
        self.loss_func = cfg.get("loss_func", "L1")
        self.precision = cfg.get("precision", "bf16")
        self.batch = int(cfg.get("micro_batch_size", 1))
        self._build_task_constants()
        self._copy = _ext.load().CopyEngine(self.device.index or 0) if self.device.type == "cuda" else None
        self._slots = [None, None]
        self._slot = 0
        self._steps_done = 0
        self._guard = self._make_guard()

    def _make_guard(self):
        """Failure detection between steps: heartbeats in the process group's store, the kernels' status word, and
        the host watchdogs of the stream waits (see ``terra_b200.runtime.watchdog``)."""
        from .runtime.watchdog import make_step_guard

        return make_step_guard(self.device, self.rank, self.world, self.model, self.optimizer)

    def _after_step(self):
        """Host-side checks where the step has synchronised anyway (the loss was just read)."""
        self._guard.after_step(self._steps_done)
        self._steps_done += 1

    # ------------------------------------------------------------------ shapes
    @property
    def local_input_shape(self):
        """Shape of this rank's model input."""
        p, C = self.archi["patch_size"], self.archi["num_channels"]
        ph, pw = self.archi["padded_shape"]
        if self.model_type == "sequential":
            return (self.batch, self.archi["height"], self.archi["width"], C)
        wp = self.manager.wp_size
        return (self.batch, ph // p // wp, pw // p, p * p * C)

    def _build_task_constants(self):
        """Land-sea mask (seeded blobs unless ``land_mask: ones``), padded, patchified and row-sliced like the input,
        and ``padding_loss_scale`` = padded area / real area (dataloader/task_specific_data.py:11-82)."""
        a = self.archi
        mask, scale = land_mask_for_rank(
            a["height"], a["width"], a["num_channels"], a["patch_size"], a["padded_shape"], a["initial_padding"],
            self.model_type, self.manager.wp_size, self.manager.wp_rank, float(self.cfg.get("land_fraction", 0.3)),
            int(self.cfg.get("land_mask_seed", 7)), self.cfg.get("land_mask", "blobs") == "ones")
        dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.task_data = {"land_sea_mask": mask.to(self.device, dt), "padding_loss_scale": scale, "test_iter_num": -1,
                          "show_gradient_flag": False}

    # ------------------------------------------------------------------ data
    def synthetic_batch(self, sample: int = 0, seed: int = 2025, pin: bool = True) -> Dict[str, torch.Tensor]:
        """This rank's slice of a seeded N(0,1) input / next-step label pair, in pinned host memory, already in
        the layout the model takes (the work the reference's data loader does on the CPU)."""
        a = self.archi
        dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        return synthetic_batch(a["height"], a["width"], a["num_channels"], a["patch_size"], a["padded_shape"],
                               a["initial_padding"], self.model_type, self.manager.wp_size, self.manager.wp_rank,
                               self.batch, sample, seed, dt, pin, "cuda" if self.device.type == "cuda" else "cpu")

    def stage(self, batch: Dict[str, torch.Tensor]):
        """Start the host->device copy of a batch on the copy engine's upload stream; returns a handle for ``step``."""
        if self._copy is None:
            return {k: v for k, v in batch.items()}
        slot = self._slot
        self._slot ^= 1
        if self._slots[slot] is None or any(self._slots[slot][k].shape != v.shape for k, v in batch.items()):
            self._slots[slot] = {k: torch.empty(v.shape, dtype=v.dtype, device=self.device) for k, v in batch.items()}
        dev = dict(self._slots[slot])
        fence = -1
        for k, v in batch.items():
            fence = self._copy.upload(v, dev[k], False)       # copies of one stream complete in order
        dev["_fence"] = fence
        return dev

    def step(self, batch: Dict[str, torch.Tensor], staged=None) -> float:
        """One optimisation step. ``batch`` holds pinned host tensors (``staged`` = handle of an earlier ``stage``
        of the same batch, so that its upload overlapped the previous step). Returns the loss (device->host read)."""
        dev = dict(staged if staged is not None else self.stage(batch))
        fence = dev.pop("_fence", -1)
        if self._copy is not None and fence >= 0:
            self._copy.wait_upload(fence)                     # only this batch's copy, not the next one's
        _, loss, _, _ = one_step_train_production(
            self.task_type, self.model_type, self.model, self.engine, self.optimizer, dev, self.task_data, self.other,
            self.precision, self.cfg.get("half_model", False), None, self.loss_func, self.gscaler, self.manager,
            self.opt_state)
        value = float(loss.item())
        self._after_step()
        return value

    def step_on_device(self, dev_batch: Dict[str, torch.Tensor]):
        """Step on tensors that already live on the device; returns the loss tensor (no host synchronisation)."""
        _, loss, _, _ = one_step_train_production(
            self.task_type, self.model_type, self.model, self.engine, self.optimizer, dev_batch, self.task_data,
            self.other, self.precision, self.cfg.get("half_model", False), None, self.loss_func, self.gscaler,
            self.manager, self.opt_state)
        return loss

    # ------------------------------------------------------------------ checkpoints, schedule
    def save_checkpoint(self, epoch: int, loss: Optional[float] = None, step: Optional[int] = None) -> Optional[str]:
        """Write ``{train_path}/{description}/ckpt/...`` in the layout the configuration implies (``single``,
        ``wp_rank``, ``rank_local``, ``fsdp_full`` or ``fsdp_sharded``: see ``terra_b200.checkpoint_io``). Collective:
        every rank calls it; returns the path this rank wrote, if any."""
        from .checkpoint_io import save_checkpoint

        return save_checkpoint(self.model, self.optimizer, loss, epoch, self.cfg.get("train_path", "./runs"),
                               self.cfg.get("description", "run"), self.model_type, self.opt_state, self.manager,
                               self.gscaler, step=step, model_config=self.cfg)

    def load_checkpoint(self, epoch: Optional[int] = None, step: Optional[int] = None):
        """Resume from a file written by ``save_checkpoint`` (or by ``train_scripts/train.py``); returns
        ``(epoch, global_step, loss)``."""
        from .checkpoint_io import load_checkpoint

        return load_checkpoint(self.model, self.optimizer, self.cfg.get("train_path", "./runs"),
                               self.cfg.get("description", "run"), self.model_type, self.opt_state, self.manager,
                               epoch=epoch, step=step, scaler=self.gscaler, model_config=self.cfg)

    def set_lr(self, lr: float) -> None:
        from .optim.utils import set_lr

        set_lr(self.optimizer, lr)

    def release(self):
        """Drop the model, optimizer and their symmetric arenas but keep the process group, so that another
        ``Trainer`` (another layout of the same job) can be built in this process."""
        self._guard.close(announce=False)
        pctx = getattr(self.model, "pctx", None)
        arena = getattr(pctx, "tp_arena", None)
        if arena is not None:
            try:
                arena.release_waits()
            except Exception:
                pass
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        self.model = self.optimizer = self._guard = self._slots = self.task_data = None

    def close(self):
        if self._guard is not None:
            self._guard.close()
        pctx = getattr(self.model, "pctx", None)
        for name in ("tp_arena",):
            arena = getattr(pctx, name, None)
            if arena is not None:
                try:
                    arena.release_waits()      # no stream may stay blocked on a peer's signal past shutdown
                except Exception:
                    pass
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
