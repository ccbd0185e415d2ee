#!/usr/bin/env bash
# The parallel layouts of the convergence experiment alone (run on every node).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
export CASES="${PARALLEL_CASES:-topo_wp topo_wp_sp topo_wp_tp topo_wp_sp_tp}"
exec bash "$here/run.sh" "$@"
