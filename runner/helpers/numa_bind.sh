#!/usr/bin/env bash
# Per-rank NUMA pinning wrapper: torchrun --no-python numa_bind.sh python3 script.py ...
# Binds the worker to the NUMA node of its GPU (read from sysfs), or round-robin when unknown.
set -euo pipefail
LOCAL_RANK="${LOCAL_RANK:-0}"
node=""
if command -v nvidia-smi >/dev/null 2>&1; then
  bus="$(nvidia-smi --query-gpu=pci.bus_id --format=csv,noheader -i "$LOCAL_RANK" 2>/dev/null | tr 'A-Z' 'a-z' | sed 's/^0000//')"
  [[ -n "$bus" && -r "/sys/bus/pci/devices/$bus/numa_node" ]] && node="$(cat "/sys/bus/pci/devices/$bus/numa_node")"
fi
if [[ -z "$node" || "$node" == "-1" ]]; then
  nn="$(numactl --hardware 2>/dev/null | awk '/available:/ {print $2}')"; nn="${nn:-1}"
  node=$(( LOCAL_RANK % nn ))
fi
if command -v numactl >/dev/null 2>&1; then exec numactl --cpunodebind="$node" --membind="$node" "$@"; else exec "$@"; fi
