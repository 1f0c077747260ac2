#!/usr/bin/env bash
# Environment presets sourced by the direct launcher: base cluster/NCCL defaults, then a per-GPU-model file.
ENV_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$ENV_DIR/base_env.sh"
GPU_MODEL="${PRIMUS_GPU_MODEL:-}"
if [[ -z "$GPU_MODEL" ]] && command -v nvidia-smi >/dev/null 2>&1; then
  GPU_MODEL="$(nvidia-smi --query-gpu=name --format=csv,noheader -i 0 2>/dev/null | awk '{print $NF}' || true)"
fi
[[ -n "$GPU_MODEL" && -f "$ENV_DIR/$GPU_MODEL.sh" ]] && source "$ENV_DIR/$GPU_MODEL.sh"
export PRIMUS_GPU_MODEL="${GPU_MODEL:-unknown}"
