#!/usr/bin/env bash
# Defaults for the fake-input correctness pair (source this, then override what differs, then run ./test_g.sh).
# One node, eight ranks, the parallel case only; the serial case is switched on with RUN_SEQ=1.
export RUN_SEQ=0 RUN_PARALLEL=1
export NUM_NODES=1 NODE_RANK=0 NPROC_PER_NODE=8 DATA_PARALLEL_SIZE=1
export MASTER_ADDR=127.0.0.1 MASTER_PORT_BASE=29731
export SCRIPT=./train_scripts/test_pretrain.py
export SEQ_MODEL_CFG=./configs/model/correctness/credit_hierarchical_swin_correctness_seq.yaml
export PARALLEL_MODEL_CFG=./configs/model/correctness/credit_hierarchical_swin_correctness_para_m1.yaml
export TERRA_USE_FAKE_INPUT=1 STEPS=4 OUT_DIR=./log/correctness
export WRITE_CSV=1 WRITE_METADATA=1 QUIET_METRICS=0 DISABLE_RANK_LOG_REDIRECT=1
export ENABLE_TORCH_PROF=0 TORCH_PROF_WRITE_TRACE=0 OMP_NUM_THREADS=1
