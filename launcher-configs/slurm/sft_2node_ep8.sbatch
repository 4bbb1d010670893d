#!/bin/bash
#SBATCH --job-name=halo-b200-sft-2node
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=64
#SBATCH --time=48:00:00
#SBATCH --output=%x-%j.out
set -euo pipefail
export CUDA_DEVICE_MAX_CONNECTIONS=1
export NVLINK_DOMAIN_SIZE=8
export HALO_NNODES=$SLURM_NNODES
export HALO_RDZV_ENDPOINT=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1):29500
RECIPE=${RECIPE:-examples/recipes/sft_moe_120b_2node_ep8.yaml}
# one launcher per node; SLURM_NODEID is that node's rank
srun bash -c 'HALO_NODE_RANK=$SLURM_NODEID python -m halo_b200.cli launch sft '"$RECIPE"' -n 8 --numa-binding'
