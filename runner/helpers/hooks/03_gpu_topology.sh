#!/usr/bin/env bash
# Global hook: record what the node looks like (GPU model, count, NVLink peer access) for the log, and refuse to
# start fused peer-memory kernels on a node whose GPUs cannot reach each other directly.
command -v nvidia-smi >/dev/null 2>&1 || exit 0
model="$(nvidia-smi --query-gpu=name --format=csv,noheader 2>/dev/null | head -1)"
count="$(nvidia-smi --query-gpu=name --format=csv,noheader 2>/dev/null | wc -l)"
[[ -n "$model" ]] && echo "env.PRIMUS_GPU_MODEL=${model// /_}" && echo "env.PRIMUS_GPU_COUNT=$count"
if (( count > 1 )); then
  if nvidia-smi topo -m 2>/dev/null | grep -q "NV[0-9]"; then
    echo "env.PRIMUS_NVLINK=1"
  else
    echo "no NVLink between the GPUs of this node: fused peer-memory kernels stay off"
    echo "env.PRIMUS_NVLINK=0"
    echo "env.PRIMUS_B200_TP_FUSED=0"
  fi
fi
