"""Worker of the multi-GPU tests: trains the small hierarchical Swin for a few steps under the layout given on the
command line and prints the losses as one JSON line (rank 0). Launched by torch.distributed.run."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def main():
    layout = json.loads(sys.argv[1])
    steps = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    from terra_b200.api import Trainer
    from terra_b200.ops.gemm import check_status

    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = dict(task_type="glorys", model_architecture="credit_hierarchical_swin", model_type="parallel", height=256,
               width=512, num_channels=32, patch_size=4, embedding_dim=128, depths=[2, 2], num_heads=[4, 8], num_layers=4,
               window_size=8, padding_policy="auto", window_assignment_mode="terra_m1_ragged_auto", precision="bf16",
               loss_func="L1", learning_rate=1e-3, optimizer_config=6 if world > 1 else 4, wp_topo=f"({world}, 1)")
    dp = int(layout.pop("dp", 1))
    if dp > 1:
        cfg["wp_topo"] = f"({world // dp}, 1)"
    cfg.update(layout)
    t = Trainer(cfg, data_parallel_group_size=dp)
    losses = []
    for i in range(steps):
        # every rank generates its own stripe of the same global field
        losses.append(t.step(t.synthetic_batch(sample=i % 2)))
    check_status(t.device)
    # Trainer.step already returns the loss reduced over the window-parallel group
    total = torch.tensor(losses, dtype=torch.float64)
    if t.rank == 0:
        print("RESULT " + json.dumps({"losses": total.tolist(), "fused_attn": t.model.pctx.fused_comm is not None,
                                      "fused_opt": getattr(t.optimizer, "fused", None) is not None,
                                      "fused_tp": getattr(getattr(t.model.pctx, "tp_comm", None), "calls", {}).get("mlp", 0) > 0,
                                      "fused_tp_attn": getattr(getattr(t.model.pctx, "tp_comm", None), "calls", {}).get("attn", 0) > 0}),
              flush=True)
    t.close()


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback

        traceback.print_exc()
        sys.stdout.flush()
        os._exit(1)          # leave at once instead of waiting in a collective the failed rank will never join
