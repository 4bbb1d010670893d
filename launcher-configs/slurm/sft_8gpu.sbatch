#!/bin/bash
#SBATCH --job-name=halo-b200-sft
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=64
#SBATCH --time=24:00:00
#SBATCH --output=%x-%j.out
set -euo pipefail
export CUDA_DEVICE_MAX_CONNECTIONS=1
export HALO_DATA_ROOT=${SLURM_TMPDIR:-/tmp}/halo_b200
RECIPE=${RECIPE:-examples/recipes/sft_moe_30b_a3b_ep8.yaml}
srun python -m halo_b200.cli launch sft "$RECIPE" -n 8 --numa-binding "$@"
