#!/bin/bash
# Multi-node training under Slurm: one torchrun per node, one process per GPU.
#   sbatch --nodes 4 examples/slurm_train.sbatch path/to/config.yaml [key=value ...]
#SBATCH --job-name=fast-llm-b200
#SBATCH --gpus-per-node=8
#SBATCH --ntasks-per-node=1
#SBATCH --cpus-per-task=96
#SBATCH --exclusive
#SBATCH --output=slurm-%j.out

set -euo pipefail
CONFIG=${1:?usage: sbatch examples/slurm_train.sbatch config.yaml [key=value ...]}
shift

MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
MASTER_PORT=${MASTER_PORT:-29500}

# The kernels are built once, in the source tree that every node sees.
srun --ntasks=1 --nodes=1 python -m fast_llm_b200.csrc.build

srun torchrun \
    --nnodes "$SLURM_JOB_NUM_NODES" --nproc-per-node 8 \
    --rdzv-backend c10d --rdzv-endpoint "$MASTER_ADDR:$MASTER_PORT" --rdzv-id "$SLURM_JOB_ID" \
    -m fast_llm_b200.cli train gpt -c "$CONFIG" "$@"
