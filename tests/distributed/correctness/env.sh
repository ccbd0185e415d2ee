#!/usr/bin/env bash
# Settings of the serial-versus-parallel convergence experiment: 2 nodes x 8 GPUs, data parallel 2, 1000 steps,
# five layouts. Source it on every node (NODE_RANK = 0 / 1, MASTER_ADDR = address of node 0), then
#   bash tests/distributed/correctness/run.sh           # all cases; finished ones are skipped on a re-run
#   python tests/distributed/correctness/analyze_correctness.py
# One 8-GPU node: NUM_NODES=1 DATA_PARALLEL_SIZE=1 SEQ_NPROC_PER_NODE=1.
export MASTER_ADDR="${MASTER_ADDR:-127.0.0.1}" MASTER_PORT_BASE="${MASTER_PORT_BASE:-29671}"
export NUM_NODES="${NUM_NODES:-2}" NODE_RANK="${NODE_RANK:-0}" NPROC_PER_NODE="${NPROC_PER_NODE:-8}"
export SEQ_NPROC_PER_NODE="${SEQ_NPROC_PER_NODE:-1}" DATA_PARALLEL_SIZE="${DATA_PARALLEL_SIZE:-2}"
export MODEL_PARALLEL_SIZE="${MODEL_PARALLEL_SIZE:-8}"
export SEQ_CASES="${SEQ_CASES:-seq_fsdp}"
export PARALLEL_CASES="${PARALLEL_CASES:-topo_wp topo_wp_sp topo_wp_tp topo_wp_sp_tp}"
export CASES="${CASES:-$SEQ_CASES $PARALLEL_CASES}"
export RUN_STEPS="${RUN_STEPS:-1000}" SKIP_FINISHED="${SKIP_FINISHED:-1}"
export MODEL_ARCHITECTURE="${MODEL_ARCHITECTURE:-credit_hierarchical_swin}"
export PATCH_SIZE="${PATCH_SIZE:-4}" WINDOW_SIZE="${WINDOW_SIZE:-8}"
export PADDED_SHAPE_H="${PADDED_SHAPE_H:-2304}" PADDED_SHAPE_W="${PADDED_SHAPE_W:-4352}"
export SMALL_EMBEDDING_DIM="${SMALL_EMBEDDING_DIM:-1024}" SMALL_NUM_LAYERS="${SMALL_NUM_LAYERS:-10}" SMALL_NUM_HEADS="${SMALL_NUM_HEADS:-8}"
export ACTIVATION_MODE="${ACTIVATION_MODE:-torch_recompute}" ACTIVATION_POLICY="${ACTIVATION_POLICY:-uniform}"
export SAMPLING_CHECKPOINT_DOWN="${SAMPLING_CHECKPOINT_DOWN:-D1}" SAMPLING_CHECKPOINT_UP="${SAMPLING_CHECKPOINT_UP:-U1}"
export RESULT_DIR="${RESULT_DIR:-./tests/distributed/correctness/results}"
export CONFIG_DIR="${CONFIG_DIR:-./tests/distributed/correctness/configs}"
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-1}"
