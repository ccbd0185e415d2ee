#!/usr/bin/env bash
# The serial baseline of the convergence experiment alone (node 0 only; the other nodes return at once).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
if [[ "${NODE_RANK:-0}" != 0 ]]; then
  echo "[run_seq.sh] NODE_RANK=${NODE_RANK}: the serial baseline runs on node 0 only"
  exit 0
fi
export NUM_NODES=1 NODE_RANK=0
export CASES="${SEQ_CASES:-seq_fsdp}"
exec bash "$here/run.sh" "$@"
