#!/usr/bin/env bash
# Global hook: PRIMUS_DETERMINISTIC=1 pins collective algorithms and turns autotuning off.
if [[ "${PRIMUS_DETERMINISTIC:-0}" == "1" ]]; then
  echo "env.NCCL_ALGO=Ring"
  echo "env.PRIMUS_B200_AUTOTUNE=0"
  echo "extra.deterministic_mode=true"
fi
