#!/usr/bin/env bash
# Defaults for every launch.  Anything already set in the environment wins.
: "${MASTER_ADDR:=127.0.0.1}"; : "${MASTER_PORT:=1234}"; : "${NNODES:=1}"; : "${NODE_RANK:=0}"; : "${GPUS_PER_NODE:=8}"
export MASTER_ADDR MASTER_PORT NNODES NODE_RANK GPUS_PER_NODE
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"
export TOKENIZERS_PARALLELISM="${TOKENIZERS_PARALLELISM:-false}"
export PYTORCH_CUDA_ALLOC_CONF="${PYTORCH_CUDA_ALLOC_CONF:-expandable_segments:True}"
# NCCL: one connection keeps kernel launch order = issue order (needed for comm/compute overlap)
export CUDA_DEVICE_MAX_CONNECTIONS="${CUDA_DEVICE_MAX_CONNECTIONS:-1}"
export TORCH_NCCL_HIGH_PRIORITY="${TORCH_NCCL_HIGH_PRIORITY:-1}"
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"
export NCCL_CHECKS_DISABLE="${NCCL_CHECKS_DISABLE:-1}"
# inter-node defaults (harmless on one node)
export NCCL_IB_GID_INDEX="${NCCL_IB_GID_INDEX:-3}"
export NCCL_CROSS_NIC="${NCCL_CROSS_NIC:-0}"
if [[ -z "${NCCL_SOCKET_IFNAME:-}" ]] && command -v ip >/dev/null 2>&1; then
  ifn="$(ip route get 1.1.1.1 2>/dev/null | awk '{for (i=1;i<=NF;i++) if ($i=="dev") {print $(i+1); exit}}')"
  [[ -n "$ifn" ]] && export NCCL_SOCKET_IFNAME="$ifn" GLOO_SOCKET_IFNAME="$ifn"
fi
# bounded waits of the fused communication kernels (cycles)
export PRIMUS_B200_WAIT_MS="${PRIMUS_B200_WAIT_MS:-1500}"
# determinism switch
if [[ "${PRIMUS_DETERMINISTIC:-0}" == "1" ]]; then
  export NCCL_ALGO="${NCCL_ALGO:-Ring}"
  export CUBLAS_WORKSPACE_CONFIG="${CUBLAS_WORKSPACE_CONFIG:-:4096:8}"
  export PRIMUS_B200_AUTOTUNE=0
fi
