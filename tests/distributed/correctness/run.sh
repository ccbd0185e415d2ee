#!/usr/bin/env bash
# Runs the cases of the convergence experiment one after the other on this node (run it on every node).
# Per case the result directory receives loss.csv, metadata.json, stdout.log and either `status.ok` or
# `failed_node<N>.txt`; with SKIP_FINISHED=1 a case that already has `status.ok` is not run again, so a failed
# sweep is resumed by re-running the same command.
set -uo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
root="$(cd "$here/../../.." && pwd)"
cd "$root"
export PYTHONPATH="$root:${PYTHONPATH:-}"
# shellcheck disable=SC1091
source "$here/env.sh"
python "$here/generate_configs.py" > /dev/null || { echo "config generation failed" >&2; exit 1; }

port="$MASTER_PORT_BASE"
overall=0
for case in $CASES; do
  port=$((port + 1))
  out="$RESULT_DIR/$case"
  mkdir -p "$out"
  if [[ "$SKIP_FINISHED" == 1 && -f "$out/status.ok" ]]; then
    echo "== $case: finished earlier, skipped"
    continue
  fi
  nproc="$NPROC_PER_NODE"
  if [[ " $SEQ_CASES " == *" $case "* ]]; then
    nproc="$SEQ_NPROC_PER_NODE"
    (( nproc * NUM_NODES >= DATA_PARALLEL_SIZE )) || nproc="$DATA_PARALLEL_SIZE"
  fi
  rm -f "$out/failed_node${NODE_RANK}.txt"
  echo "== $case: node $NODE_RANK of $NUM_NODES, $nproc ranks here, port $port"
  python -m torch.distributed.run --master_addr "$MASTER_ADDR" --master_port "$port" --nnodes "$NUM_NODES" \
      --node_rank "$NODE_RANK" --nproc_per_node "$nproc" train_scripts/test_pretrain.py \
      --data_parallel_group_size "$DATA_PARALLEL_SIZE" --model_cfg "$CONFIG_DIR/correctness_${case}.yaml" \
      --steps "$RUN_STEPS" --metrics_csv "$out/loss.csv" --metrics_json "$out/metadata.json" \
      --disable_rank_log_redirect --disable_torch_prof > "$out/stdout_node${NODE_RANK}.log" 2>&1
  rc=$?
  if (( rc == 0 )); then
    [[ "$NODE_RANK" == 0 ]] && date -u +%FT%TZ > "$out/status.ok"
  else
    echo "exit code $rc at $(date -u +%FT%TZ)" > "$out/failed_node${NODE_RANK}.txt"
    echo "== $case: FAILED (exit $rc), see $out/stdout_node${NODE_RANK}.log" >&2
    overall=1
  fi
done
exit "$overall"
