#!/bin/bash
#SBATCH --job-name=kfb200-13b-val
#SBATCH --partition=<partition>
#SBATCH --account=<account>
#SBATCH --nodes=4
#SBATCH --ntasks-per-node=8
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=12
#SBATCH --mem=0
#SBATCH --time=02:00:00
#SBATCH --output=logs/%j_%x.out
#
# Short 13B validation run: TP inside the node, sharded data parallel across nodes,
# 200 steps with profiling of steps 20-25 and a checkpoint at the end.
# Parity: scripts/slurm/13b_validation.sh in the reference.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$HERE/_env.sh"
kf_export_env
CONFIG="${1:-configs/train/13b_24gpu_validation.toml}"; shift || true
kf_banner "13b validation, ${CONFIG}"
srun --kill-on-bad-exit=1 "$HERE/_run_training.sh" "${CONFIG}" \
    --train.max_steps=200 --profiling.enable=true --profiling.start_step=20 --profiling.end_step=25 \
    --checkpoint.interval=200 "$@"
