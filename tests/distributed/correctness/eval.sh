#!/usr/bin/env bash
# Compares the finished cases with the baseline: summary.csv, report.md and the loss plots (or loss_delta.csv) in the
# result directory. Extra arguments go to analyze_correctness.py (e.g. --tolerance 1e-2).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
root="$(cd "$here/../../.." && pwd)"
cd "$root"
# shellcheck disable=SC1091
source "$here/env.sh"
# shellcheck disable=SC2086
exec python "$here/analyze_correctness.py" --result_dir "$RESULT_DIR" --config_dir "$CONFIG_DIR" \
    --baseline "${BASELINE:-seq_fsdp}" --cases $CASES "$@"
