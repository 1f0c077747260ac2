#!/usr/bin/env bash
# Global hook: choose NCCL's network settings when the user did not.  Multi-node: list the InfiniBand / RoCE
# devices under /sys/class/infiniband for NCCL_IB_HCA and pick the interface of the default route for the bootstrap
# socket; single node: nothing to choose (NVLink / NVSwitch carries everything), only keep NVLS on.
nnodes="${NNODES:-1}"
if [[ -z "${NCCL_SOCKET_IFNAME:-}" ]]; then
  ifname="$(ip -o -4 route show to default 2>/dev/null | awk '{print $5; exit}')"
  [[ -n "$ifname" ]] && echo "env.NCCL_SOCKET_IFNAME=$ifname" && echo "env.GLOO_SOCKET_IFNAME=$ifname"
fi
if (( nnodes > 1 )) && [[ -z "${NCCL_IB_HCA:-}" && -d /sys/class/infiniband ]]; then
  hcas="$(ls /sys/class/infiniband 2>/dev/null | paste -sd, -)"
  if [[ -n "$hcas" ]]; then
    echo "env.NCCL_IB_HCA=$hcas"
  else
    echo "no InfiniBand / RoCE device found: NCCL will use sockets between nodes"
    echo "env.NCCL_IB_DISABLE=1"
  fi
fi
if (( nnodes == 1 )) && [[ -z "${NCCL_NVLS_ENABLE:-}" ]]; then
  echo "env.NCCL_NVLS_ENABLE=1"
fi
