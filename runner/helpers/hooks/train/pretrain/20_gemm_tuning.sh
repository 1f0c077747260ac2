#!/usr/bin/env bash
# Stage hook (train pretrain): GEMM tile tuning workflow, driven by PRIMUS_GEMM_TUNING=1 and PRIMUS_GEMM_TUNING_STAGE.
#   stage 1  dump the GEMM shapes of this (short) job to $PRIMUS_GEMM_TUNING_DIR/gemm_shape/
#   stage 2  offline: python -m primus_b200.tools.tune_gemm --shapes <dir>/gemm_shape/*.json --out <dir>/gemm_tune/tuned.json
#   stage 3  train with the tuned table
# Off under PRIMUS_DETERMINISTIC=1.
[[ "${PRIMUS_GEMM_TUNING:-0}" == "1" ]] || exit 0
if [[ "${PRIMUS_DETERMINISTIC:-0}" == "1" ]]; then
  echo "GEMM tuning is off in deterministic mode"
  exit 0
fi
dir="${PRIMUS_GEMM_TUNING_DIR:-./output/gemm_tuning}"
case "${PRIMUS_GEMM_TUNING_STAGE:-0}" in
  1)
    mkdir -p "$dir/gemm_shape"
    echo "env.PRIMUS_B200_GEMM_TUNING_STAGE=1"
    echo "env.PRIMUS_B200_GEMM_SHAPE_DIR=$dir/gemm_shape"
    echo "GEMM tuning stage 1: shapes go to $dir/gemm_shape"
    ;;
  2)
    echo "GEMM tuning stage 2 runs offline: python -m primus_b200.tools.tune_gemm --shapes '$dir/gemm_shape/*.json' --out $dir/gemm_tune/tuned.json"
    ;;
  3)
    if [[ -f "$dir/gemm_tune/tuned.json" ]]; then
      echo "env.PRIMUS_B200_GEMM_TUNING_FILE=$dir/gemm_tune/tuned.json"
      echo "GEMM tuning stage 3: using $dir/gemm_tune/tuned.json"
    else
      echo "GEMM tuning stage 3: $dir/gemm_tune/tuned.json not found, running with the built-in tile heuristic"
    fi
    ;;
  *) ;;
esac
