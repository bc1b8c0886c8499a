#!/bin/bash
# Multi-node pre-training under SLURM: one task per GPU, rendezvous through rank 0's host.
# Run inside an allocation, e.g.
#   srun --ntasks-per-node=8 --gpus-per-node=8 multiprocess_pretrain_slurm.sh xxl 128 /ckpt/run1
# Every task passes the flags the reference's GPU scripts pass (--multiprocess_gpu,
# --coordinator_address, --process_count, --process_index).
set -euo pipefail
SIZE=${1:?model size}; BATCH=${2:?global batch}; MODEL_DIR=${3:?model dir}; STEPS=${4:-1000}
shift $(( $# < 4 ? $# : 4 ))
HEAD=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n1)
export LOCAL_RANK=${SLURM_LOCALID}
exec python -m t5x_b200.train --multiprocess_gpu \
  --coordinator_address="${HEAD}:${MASTER_PORT:-29400}" \
  --process_count="${SLURM_NTASKS}" --process_index="${SLURM_PROCID}" \
  --gin_file="t5x/examples/t5/t5_1_1/${SIZE}.gin" \
  --gin_file="t5x/configs/runs/pretrain.gin" \
  --gin.MODEL_DIR="\"${MODEL_DIR}\"" \
  --gin.MIXTURE_OR_TASK_NAME="\"${TASK:-synthetic_span_corruption}\"" \
  --gin.TASK_FEATURE_LENGTHS="{'inputs': 512, 'targets': 114}" \
  --gin.USE_CACHED_TASKS=False --gin.DROPOUT_RATE=0.0 \
  --gin.BATCH_SIZE="${BATCH}" --gin.TRAIN_STEPS="${STEPS}" "$@"
