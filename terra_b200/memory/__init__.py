"""Memory orchestration: activation recompute, pinned-host boundary offload, checkpoint scheduling."""
