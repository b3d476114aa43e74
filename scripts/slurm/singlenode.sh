#!/bin/bash
#SBATCH --job-name=kfb200-1node
#SBATCH --partition=<partition>
#SBATCH --account=<account>
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=96
#SBATCH --mem=0
#SBATCH --time=24:00:00
#SBATCH --output=logs/%j_%x.out
#SBATCH --signal=B:SIGTERM@120
#
# One node, every GPU of it, via torchrun.
#   sbatch scripts/slurm/singlenode.sh configs/train/7b.toml --train.max_steps=1000
#   NGPUS=4 sbatch --gpus-per-node=4 scripts/slurm/singlenode.sh configs/train/debug.toml
# Parity: scripts/slurm/singlenode.sh in the reference.
set -euo pipefail
CONFIG="${1:?usage: singlenode.sh <config.toml> [--section.key=value ...]}"; shift
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$HERE/_env.sh"
kf_export_env
NGPUS="${NGPUS:-${SLURM_GPUS_ON_NODE:-8}}"
kf_banner "single node, ${NGPUS} GPUs, ${CONFIG} $*"
cd "$HERE/../.."
python -c "from kempnerforge_b200.ops.build import build; build()"
# torchrun forwards SIGTERM to the ranks; the trainer then writes an emergency checkpoint.
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NGPUS}" \
    --master-addr 127.0.0.1 --master-port "${MASTER_PORT}" \
    scripts/train.py "${CONFIG}" "$@"
