#!/bin/bash
# Samples DCGM counters on this node once a second into a CSV while a job runs:
#   scripts/slurm/_dcgm_monitor.sh logs/dcgm_${SLURM_JOB_ID}_$(hostname).csv &
# Fields: 203 GPU util, 1002 SM active, 1003 SM occupancy, 1004 tensor pipe active,
# 1005 DRAM active, 252 framebuffer used, 155 power, 150 temperature, 1011/1012 NVLink tx/rx bytes.
# Read-only: it changes no setting of any GPU. Parity: scripts/slurm/_dcgm_monitor.sh:245-248.
set -euo pipefail
OUT="${1:-logs/dcgm_$(hostname).csv}"
mkdir -p "$(dirname "$OUT")"
if ! command -v dcgmi >/dev/null 2>&1; then
    echo "dcgmi not found; falling back to nvidia-smi sampling" >&2
    exec nvidia-smi --query-gpu=timestamp,index,utilization.gpu,memory.used,power.draw,temperature.gpu,clocks.sm \
        --format=csv -lms 1000 > "$OUT"
fi
exec dcgmi dmon -e 203,1002,1003,1004,1005,252,155,150,1011,1012 -d 1000 > "$OUT"
