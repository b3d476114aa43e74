#!/bin/bash
#SBATCH --job-name=kfb200-mfu_scaling
#SBATCH --partition=<partition>
#SBATCH --account=<account>
#SBATCH --nodes=4
#SBATCH --ntasks-per-node=8
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=12
#SBATCH --mem=0
#SBATCH --time=04:00:00
#SBATCH --output=logs/%j_%x.out
#
# Runs the "mfu_scaling" experiment matrix (benchmarks/cluster_bench.py) inside this allocation, or on the
# local node when started by hand. STEPS and DATA_ARGS may be set in the environment, e.g.
#   DATA_ARGS="--data.dataset_path=/data/fineweb-edu-llama3" STEPS=50 sbatch mfu_bench.sh
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$HERE/../../scripts/slurm/_env.sh"
kf_export_env
cd "$HERE/../.."
exec python benchmarks/cluster_bench.py mfu_scaling --steps "${STEPS:-30}" --extra "${DATA_ARGS:-}" \
    --results-dir "benchmarks/results/mfu_scaling" "$@"
