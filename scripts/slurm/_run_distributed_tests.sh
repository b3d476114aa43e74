#!/bin/bash
# Runs the multi-rank test files. CPU ranks (gloo) need no allocation:
#   scripts/slurm/_run_distributed_tests.sh cpu
# GPU ranks, one node:
#   scripts/slurm/_run_distributed_tests.sh gpu
# Parity: scripts/slurm/_run_distributed_tests.sh in the reference (there pytest itself is the
# rank under torchrun; here each test spawns its own ranks, so plain pytest is enough).
set -euo pipefail
MODE="${1:-cpu}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
cd "$HERE/../.."
export MASTER_ADDR=127.0.0.1
case "$MODE" in
    cpu) exec python -m pytest tests/test_distributed_cpu.py -q -m "not gpu" ;;
    gpu) export NCCL_NVLS_ENABLE=0
         exec python -m pytest tests/test_multi_gpu.py -q -m gpu ;;
    *)   echo "unknown mode '$MODE' (cpu|gpu)"; exit 2 ;;
esac
