#!/bin/bash
# One rank of a multi-node job: maps SLURM's task ids to the torch.distributed
# environment and runs the trainer. Launched by `srun` from multinode.sh / 7b_requeue.sh.
# Parity: scripts/slurm/_run_training.sh in the reference.
set -euo pipefail
export RANK="${SLURM_PROCID:?run under srun}"
export LOCAL_RANK="${SLURM_LOCALID}"
export WORLD_SIZE="${SLURM_NTASKS}"
export LOCAL_WORLD_SIZE="${SLURM_NTASKS_PER_NODE:-8}"
REPO="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
cd "$REPO"
# The native library is built once per node by local rank 0; the others wait for the stamp.
if [[ "$LOCAL_RANK" == "0" ]]; then
    python -c "from kempnerforge_b200.ops.build import build; build()"
else
    # bounded: if local rank 0's build fails there will never be a stamp, and the job must end, not hang
    for _ in $(seq 1 "${KF_BUILD_WAIT_SEC:-900}"); do
        [[ -f kempnerforge_b200/lib/build.stamp ]] && break
        sleep 1
    done
    [[ -f kempnerforge_b200/lib/build.stamp ]] || { echo "native library was not built on this node" >&2; exit 1; }
fi
exec python scripts/train.py "$@"
