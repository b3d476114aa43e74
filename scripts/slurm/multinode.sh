#!/bin/bash
#SBATCH --job-name=kfb200
#SBATCH --partition=<partition>
#SBATCH --account=<account>
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=8
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=12
#SBATCH --mem=0
#SBATCH --time=48:00:00
#SBATCH --output=logs/%j_%x.out
#SBATCH --signal=B:SIGTERM@120
#SBATCH --requeue
#
# Many nodes, one srun task per GPU (--ntasks-per-node must equal --gpus-per-node).
#   sbatch --nodes=4 scripts/slurm/multinode.sh configs/train/7b.toml --train.max_steps=50000
# SIGTERM arrives 120 s before the limit or a preemption; the trainer checkpoints and exits,
# SLURM requeues the job, and the next incarnation resumes from the `latest` checkpoint.
# Parity: scripts/slurm/multinode.sh:13-14,41-91 in the reference.
set -euo pipefail
CONFIG="${1:?usage: multinode.sh <config.toml> [--section.key=value ...]}"; shift
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$HERE/_env.sh"
kf_export_env
kf_banner "multi node, $(( SLURM_NNODES * ${SLURM_NTASKS_PER_NODE:-8} )) GPUs, ${CONFIG} $*"
srun --kill-on-bad-exit=1 "$HERE/_run_training.sh" "${CONFIG}" "$@"
