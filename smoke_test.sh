#!/usr/bin/env bash
# Quick health check without a GPU: the CPU unit tests and a byte-compile of the modules every entry point imports.
set -euo pipefail
cd "$(dirname "${BASH_SOURCE[0]}")"
python -m pytest -q tests/test_window_assignment.py tests/test_config_and_memory.py
python -m py_compile terra_b200/parallel/window_assignment.py terra_b200/models/get_model.py terra_b200/ops/attention.py \
  terra_b200/api.py bench.py __graft_entry__.py
echo "smoke test: ok"
