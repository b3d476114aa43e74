#!/bin/bash
# Run inside an interactive allocation (salloc / srun --pty) or on a workstation:
#   scripts/slurm/interactive.sh configs/train/debug.toml [--section.key=value ...]
#   NGPUS=2 scripts/slurm/interactive.sh configs/train/debug_moe.toml
# Uses every visible GPU unless NGPUS is set. Parity: scripts/slurm/interactive.sh in the reference.
set -euo pipefail
CONFIG="${1:?usage: interactive.sh <config.toml> [overrides]}"; shift
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$HERE/_env.sh"
kf_export_env
export MASTER_ADDR=127.0.0.1
if [[ -z "${NGPUS:-}" ]]; then
    NGPUS=$(python -c "import torch; print(max(torch.cuda.device_count(), 1))")
fi
kf_banner "interactive, ${NGPUS} process(es), ${CONFIG} $*"
cd "$HERE/../.."
python -c "from kempnerforge_b200.ops.build import build; build()" || true
if [[ "$NGPUS" == "1" ]]; then
    exec python scripts/train.py "${CONFIG}" "$@"
fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NGPUS}" \
    --master-addr 127.0.0.1 --master-port "${MASTER_PORT}" scripts/train.py "${CONFIG}" "$@"
