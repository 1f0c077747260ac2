#!/usr/bin/env bash
# B200 (HGX, NVSwitch) node preset.
export NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-1}"      # in-switch reductions
export NCCL_CUMEM_ENABLE="${NCCL_CUMEM_ENABLE:-1}"
export NCCL_P2P_NET_CHUNKSIZE="${NCCL_P2P_NET_CHUNKSIZE:-524288}"
export PRIMUS_B200_SYMM_HEAP_MB="${PRIMUS_B200_SYMM_HEAP_MB:-2048}"
