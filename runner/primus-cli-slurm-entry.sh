#!/usr/bin/env bash
# Per-node entry under Slurm: derive the torchrun topology from Slurm's variables, then run a mode.
set -euo pipefail
RUNNER_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$RUNNER_DIR/lib/common.sh"
source "$RUNNER_DIR/lib/validation.sh"
validate_slurm_env
export NNODES="${SLURM_NNODES:-${SLURM_JOB_NUM_NODES:-1}}"
export NODE_RANK="${SLURM_NODEID:-0}"
if [[ -z "${MASTER_ADDR:-}" ]]; then
  if command -v scontrol >/dev/null 2>&1 && [[ -n "${SLURM_JOB_NODELIST:-}" ]]; then
    MASTER_ADDR="$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n1)"
  else
    MASTER_ADDR="127.0.0.1"
  fi
fi
export MASTER_ADDR
export MASTER_PORT="${MASTER_PORT:-$(( 20000 + ${SLURM_JOB_ID:-0} % 20000 ))}"
export GPUS_PER_NODE="${GPUS_PER_NODE:-${SLURM_GPUS_ON_NODE:-8}}"
LOG_INFO "slurm entry: node $NODE_RANK/$NNODES master $MASTER_ADDR:$MASTER_PORT gpus $GPUS_PER_NODE"
exec bash "$RUNNER_DIR/primus-cli" "$@"
