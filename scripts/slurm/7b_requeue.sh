#!/bin/bash
#SBATCH --job-name=kfb200-7b
#SBATCH --partition=<partition>
#SBATCH --account=<account>
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=8
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=12
#SBATCH --mem=0
#SBATCH --time=08:00:00
#SBATCH --output=logs/%j_%x.out
#SBATCH --signal=B:SIGTERM@120
#SBATCH --requeue
#SBATCH --open-mode=append
#
# Long Llama-3-8B-shape run cut into time-limited segments: each segment ends with an
# emergency checkpoint on SIGTERM and the job requeues itself until max_steps is reached.
# Parity: scripts/slurm/7b_requeue.sh in the reference.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$HERE/_env.sh"
kf_export_env
CONFIG="${CONFIG:-configs/train/7b_16gpu_fp8.toml}"
CKPT_DIR="${CKPT_DIR:-checkpoints/7b_requeue}"
kf_banner "requeue-able 7b run, segment ${SLURM_RESTART_COUNT:-0}, checkpoints in ${CKPT_DIR}"
set +e
srun --kill-on-bad-exit=1 "$HERE/_run_training.sh" "${CONFIG}" \
    --checkpoint.dir="${CKPT_DIR}" --checkpoint.interval=500 "$@"
rc=$?
set -e
if [[ $rc -ne 0 && -e "${CKPT_DIR}/latest" ]]; then
    echo "segment ended with rc=${rc}; asking SLURM to requeue ${SLURM_JOB_ID}"
    scontrol requeue "${SLURM_JOB_ID}"
fi
exit $rc
