#!/usr/bin/env bash
# Runs the serial and / or the parallel correctness case of test_pretrain.py under torch.distributed.run.
#   ./test_g.sh [node_rank]      (environment: see test_env.sh; every variable has the same default here)
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
cd "$here"
export PYTHONPATH="$here:${PYTHONPATH:-}"

: "${NUM_NODES:=1}" "${NPROC_PER_NODE:=8}" "${DATA_PARALLEL_SIZE:=1}"
: "${MASTER_ADDR:=127.0.0.1}" "${MASTER_PORT_BASE:=29731}" "${RUN_SEQ:=0}" "${RUN_PARALLEL:=1}"
: "${SCRIPT:=./train_scripts/test_pretrain.py}" "${STEPS:=4}" "${OUT_DIR:=./log/correctness}"
: "${SEQ_MODEL_CFG:=./configs/model/correctness/credit_hierarchical_swin_correctness_seq.yaml}"
: "${PARALLEL_MODEL_CFG:=./configs/model/correctness/credit_hierarchical_swin_correctness_para_m1.yaml}"
: "${WRITE_CSV:=1}" "${WRITE_METADATA:=1}" "${QUIET_METRICS:=0}" "${DISABLE_RANK_LOG_REDIRECT:=1}" "${ENABLE_TORCH_PROF:=0}"
NODE_RANK="${1:-${NODE_RANK:-0}}"

die() { echo "test_g.sh: $*" >&2; exit 1; }
(( NODE_RANK >= 0 && NODE_RANK < NUM_NODES )) || die "NODE_RANK=${NODE_RANK} outside [0, ${NUM_NODES})"
(( (NUM_NODES * NPROC_PER_NODE) % DATA_PARALLEL_SIZE == 0 )) || die "world size not divisible by DATA_PARALLEL_SIZE"
for f in "$SCRIPT" "$SEQ_MODEL_CFG" "$PARALLEL_MODEL_CFG"; do [[ -f "$f" ]] || die "missing file $f"; done

launch() {   # launch <case name> <port> <ranks on this node> <config>
  local out="${OUT_DIR}/$(echo "$1" | tr '[:upper:]' '[:lower:]')"
  mkdir -p "$out"
  local -a extra=(--data_parallel_group_size "$DATA_PARALLEL_SIZE" --model_cfg "$4" --steps "$STEPS")
  [[ "$WRITE_CSV" == 1 ]] && extra+=(--metrics_csv "$out/loss.csv")
  if [[ "$WRITE_METADATA" == 1 ]]; then extra+=(--metrics_json "$out/metadata.json"); else extra+=(--metrics_no_json); fi
  [[ "$QUIET_METRICS" == 1 ]] && extra+=(--quiet_metrics)
  [[ "$DISABLE_RANK_LOG_REDIRECT" == 1 ]] && extra+=(--disable_rank_log_redirect)
  [[ "$ENABLE_TORCH_PROF" == 0 ]] && extra+=(--disable_torch_prof)
  echo "== $1: node ${NODE_RANK} of ${NUM_NODES}, $3 ranks here"
  python -m torch.distributed.run --master_addr "$MASTER_ADDR" --master_port "$2" --nnodes "$NUM_NODES" \
    --node_rank "$NODE_RANK" --nproc_per_node "$3" "$SCRIPT" "${extra[@]}"
}

if [[ "$RUN_SEQ" == 1 ]]; then
  (( DATA_PARALLEL_SIZE % NUM_NODES == 0 )) || die "the serial case needs DATA_PARALLEL_SIZE divisible by NUM_NODES"
  launch SEQ "$MASTER_PORT_BASE" "$(( DATA_PARALLEL_SIZE / NUM_NODES ))" "$SEQ_MODEL_CFG"
fi
if [[ "$RUN_PARALLEL" == 1 ]]; then
  launch PARALLEL "$(( MASTER_PORT_BASE + 1 ))" "$NPROC_PER_NODE" "$PARALLEL_MODEL_CFG"
fi
