#!/bin/bash
# Multi-node launch under SLURM: one torchrun agent per node, one process per GPU, rendezvous on the first node.
#
#   sbatch --nodes=4 multinode_trainer.slurm
#   MODULE=llama3 CONFIG=llama3_70b sbatch --nodes=8 multinode_trainer.slurm --parallelism.tensor_parallel_degree 8
#
# Extra arguments are passed to the trainer as config overrides.
#SBATCH --job-name=torchtitan_b200
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=96
#SBATCH --exclusive

set -euo pipefail

MODULE=${MODULE:-llama3}
CONFIG=${CONFIG:-llama3_8b}
GPUS_PER_NODE=${GPUS_PER_NODE:-8}
TRAIN_FILE=${TRAIN_FILE:-torchtitan_b200.train}

nodes=( $(scontrol show hostnames "$SLURM_JOB_NODELIST") )
head_node=${nodes[0]}
head_ip=$(srun --nodes=1 --ntasks=1 -w "$head_node" hostname --ip-address | awk '{print $1}')
echo "head node ${head_node} (${head_ip}), ${SLURM_NNODES} nodes x ${GPUS_PER_NODE} GPUs"

export PYTORCH_ALLOC_CONF=${PYTORCH_ALLOC_CONF:-expandable_segments:True}
export LOGLEVEL=${LOGLEVEL:-INFO}
# NVLink peer-memory paths work inside a node; across nodes the sharded axes fall back to NCCL
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}

srun python -m torch.distributed.run \
    --nnodes "${SLURM_NNODES}" --nproc-per-node "${GPUS_PER_NODE}" \
    --rdzv-id "${SLURM_JOB_ID}" --rdzv-backend c10d --rdzv-endpoint "${head_ip}:29500" \
    --local-ranks-filter 0 --role rank --tee 3 \
    -m "${TRAIN_FILE}" --module "${MODULE}" --config "${CONFIG}" "$@"
