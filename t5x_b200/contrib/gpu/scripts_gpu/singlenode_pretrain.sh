#!/bin/bash
# Pre-train a T5.1.1 model on the GPUs of one machine: one process per GPU under torchrun.
#
#   singlenode_pretrain.sh <size: small|base|large|xl|xxl> <num gpus> <global batch> \
#       <model dir> [train steps] [extra --gin.* flags ...]
#
# Data parallel with the optimizer sharded over replicas is the default; add
# --gin.partitioning.PjitPartitioner.num_partitions=N for N-way tensor parallelism.
set -euo pipefail
SIZE=${1:?model size}; NGPU=${2:?number of gpus}; BATCH=${3:?global batch}; MODEL_DIR=${4:?model dir}
STEPS=${5:-1000}
shift $(( $# < 5 ? $# : 5 ))
export NCCL_NVLS_ENABLE=${NCCL_NVLS_ENABLE:-1}
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" \
  --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29400}" \
  -m t5x_b200.train --multiprocess_gpu \
  --gin_file="t5x/examples/t5/t5_1_1/${SIZE}.gin" \
  --gin_file="t5x/configs/runs/pretrain.gin" \
  --gin.MODEL_DIR="\"${MODEL_DIR}\"" \
  --gin.MIXTURE_OR_TASK_NAME="\"${TASK:-synthetic_span_corruption}\"" \
  --gin.TASK_FEATURE_LENGTHS="{'inputs': 512, 'targets': 114}" \
  --gin.USE_CACHED_TASKS=False \
  --gin.DROPOUT_RATE=0.0 \
  --gin.BATCH_SIZE="${BATCH}" \
  --gin.TRAIN_STEPS="${STEPS}" \
  "$@"
