# Sourced by the launchers in this directory: rendezvous, network and logging
# environment for one-process-per-GPU jobs on 8x B200 (NVLink 5 / NVSwitch) nodes.
# Parity: the reference exports the same variables inline in each script
# (scripts/slurm/multinode.sh:41-70, scripts/slurm/singlenode.sh).

kf_pick_port() {
    # A free TCP port derived from the job id first (stable across ranks), checked against
    # listening sockets; falls back to the next free one.
    local base=$(( 15000 + (${SLURM_JOB_ID:-$$} % 5000) ))
    local used
    used=$(ss -Htan 2>/dev/null | awk '{print $4}' | sed 's/.*://' | sort -un)
    local p=$base
    while echo "$used" | grep -qx "$p"; do p=$((p + 1)); done
    echo "$p"
}

kf_fabric_ifname() {
    # First interface that is UP with an address among InfiniBand / RoCE style names.
    local name
    name=$(ip -br addr 2>/dev/null | awk '$2=="UP" && $3!="" && $1 ~ /^(ib|ibp|mlx|roce)[0-9a-z]*/ {print $1; exit}')
    echo "${name:-}"
}

kf_export_env() {
    local nodes_first
    if [[ -n "${SLURM_JOB_NODELIST:-}" ]]; then
        nodes_first=$(scontrol show hostnames "${SLURM_JOB_NODELIST}" | head -n 1)
    else
        nodes_first=127.0.0.1
    fi
    export MASTER_ADDR="${MASTER_ADDR:-$nodes_first}"
    export MASTER_PORT="${MASTER_PORT:-$(kf_pick_port)}"

    local ifn
    ifn=$(kf_fabric_ifname)
    if [[ -n "$ifn" ]]; then
        export NCCL_SOCKET_IFNAME="${NCCL_SOCKET_IFNAME:-$ifn}"
        export GLOO_SOCKET_IFNAME="${GLOO_SOCKET_IFNAME:-$ifn}"
        export NCCL_IB_DISABLE="${NCCL_IB_DISABLE:-0}"
        export NCCL_NET_GDR_LEVEL="${NCCL_NET_GDR_LEVEL:-2}"
    fi
    # Inside a node every pair of GPUs talks through NVSwitch; let NCCL use in-switch reduction.
    export NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-1}"
    export TORCH_NCCL_ASYNC_ERROR_HANDLING="${TORCH_NCCL_ASYNC_ERROR_HANDLING:-1}"
    export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"
    mkdir -p logs
}

kf_banner() {
    echo "== kempnerforge_b200 :: $1"
    echo "   job=${SLURM_JOB_ID:-local} nodes=${SLURM_NNODES:-1} (${SLURM_JOB_NODELIST:-localhost}) restart=${SLURM_RESTART_COUNT:-0}"
    echo "   rendezvous=${MASTER_ADDR}:${MASTER_PORT} fabric_if=${NCCL_SOCKET_IFNAME:-default}"
}
