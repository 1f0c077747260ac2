#!/usr/bin/env bash
# primus-cli direct: launch on this host (or inside the current container) with torchrun.
#
#   primus-cli direct [--env K=V]... [--env-file F] [--script PY] [--patch SH]... [--log_file F]
#                     [--numa|--no-numa] [--single] [--silent] [--gpus N] [--nnodes N] [--node_rank R]
#                     [--master_addr A] [--master_port P] -- <primus args>
#
# Topology comes from flags, then the environment (NNODES / NODE_RANK / MASTER_ADDR / MASTER_PORT /
# GPUS_PER_NODE), then Slurm variables when inside an allocation, then .primus.yaml `direct.*`.
# Before launching: environment presets (helpers/envs), hooks (helpers/hooks, protocol: a hook prints
# `env.KEY=VALUE` to export a variable or `extra.name=value` to append `--name value` to the primus
# arguments) and patch scripts (--patch) run in that order.
set -euo pipefail

RUNNER_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
export PRIMUS_ROOT="${PRIMUS_ROOT:-$(cd "$RUNNER_DIR/.." && pwd)}"
source "$RUNNER_DIR/lib/common.sh"
source "$RUNNER_DIR/lib/config.sh"
source "$RUNNER_DIR/lib/validation.sh"
load_config_auto "$RUNNER_DIR" "${PRIMUS_CLI_CONFIG_FILE:-}" || exit 2

SCRIPT="$(cfg_get direct.script primus_b200/cli/main.py)"
LOG_FILE="$(cfg_get direct.log_file "")"
NUMA="$(cfg_get direct.numa auto)"
SINGLE=0
PATCHES=()
ENV_ASSIGN=()
CLI_GPUS="" CLI_NNODES="" CLI_NODE_RANK="" CLI_MASTER_ADDR="" CLI_MASTER_PORT=""
PRIMUS_ARGS=()

while [[ $# -gt 0 ]]; do
  case "$1" in
    --env) [[ $# -ge 2 ]] || usage_error "--env needs KEY=VALUE"; validate_env_assignment "$2"; ENV_ASSIGN+=("$2"); shift 2 ;;
    --env-file) validate_file "$2" "env file"; while IFS= read -r l; do [[ -z "$l" || "$l" == \#* ]] || { validate_env_assignment "$l"; ENV_ASSIGN+=("$l"); }; done < "$2"; shift 2 ;;
    --script) SCRIPT="$2"; shift 2 ;;
    --patch) PATCHES+=("$2"); shift 2 ;;
    --log_file|--log-file) LOG_FILE="$2"; shift 2 ;;
    --numa) NUMA=on; shift ;;
    --no-numa) NUMA=off; shift ;;
    --single) SINGLE=1; shift ;;
    --silent) export PRIMUS_SILENT=1; shift ;;
    --gpus|--gpus_per_node) CLI_GPUS="$2"; shift 2 ;;
    --nnodes) CLI_NNODES="$2"; shift 2 ;;
    --node_rank) CLI_NODE_RANK="$2"; shift 2 ;;
    --master_addr) CLI_MASTER_ADDR="$2"; shift 2 ;;
    --master_port) CLI_MASTER_PORT="$2"; shift 2 ;;
    -h|--help) sed -n '2,14p' "${BASH_SOURCE[0]}" | sed 's/^# \{0,1\}//'; exit 0 ;;
    --) shift; PRIMUS_ARGS=("$@"); break ;;
    *) usage_error "unknown option for direct mode: $1 (did you forget '--' before the primus arguments?)" ;;
  esac
done
[[ ${#PRIMUS_ARGS[@]} -gt 0 ]] || usage_error "no primus arguments given (expected: -- train pretrain --config ...)"

for kv in "${ENV_ASSIGN[@]:-}"; do [[ -n "$kv" ]] && export "${kv?}"; done

# ---- topology: flags > environment > Slurm > defaults file
if [[ -n "${SLURM_JOB_ID:-}" && -z "${NNODES:-}" ]]; then
  export NNODES="${SLURM_NNODES:-1}"
  export NODE_RANK="${SLURM_NODEID:-0}"
  if [[ -z "${MASTER_ADDR:-}" ]] && command -v scontrol >/dev/null 2>&1; then
    MASTER_ADDR="$(scontrol show hostnames "${SLURM_JOB_NODELIST:-}" 2>/dev/null | head -n1 || true)"
    export MASTER_ADDR
  fi
fi
export GPUS_PER_NODE="${CLI_GPUS:-${GPUS_PER_NODE:-$(cfg_get direct.gpus_per_node 8)}}"
export NNODES="${CLI_NNODES:-${NNODES:-1}}"
export NODE_RANK="${CLI_NODE_RANK:-${NODE_RANK:-0}}"
export MASTER_ADDR="${CLI_MASTER_ADDR:-${MASTER_ADDR:-127.0.0.1}}"
export MASTER_PORT="${CLI_MASTER_PORT:-${MASTER_PORT:-$(cfg_get direct.master_port 1234)}}"

# node_smoke and other single-process commands never need torchrun
case "${PRIMUS_ARGS[0]}" in node_smoke|projection|data) [[ "${PRIMUS_ARGS[0]}" == "node_smoke" ]] && SINGLE=1 ;; esac
validate_distributed_params

# ---- environment presets
# shellcheck source=helpers/envs/primus-env.sh
source "$RUNNER_DIR/helpers/envs/primus-env.sh"

# ---- hooks: group = first primus arg (train / benchmark ...), name = second (pretrain ...)
HOOK_EXTRA_ARGS=()
# shellcheck source=helpers/execute_hooks.sh
source "$RUNNER_DIR/helpers/execute_hooks.sh"
execute_hooks "${PRIMUS_ARGS[0]}" "${PRIMUS_ARGS[1]:-}" "${PRIMUS_ARGS[@]}"
PRIMUS_ARGS+=("${HOOK_EXTRA_ARGS[@]:-}")
# drop the empty element bash adds when the array was empty
TMP=(); for a in "${PRIMUS_ARGS[@]}"; do [[ -n "$a" ]] && TMP+=("$a"); done; PRIMUS_ARGS=("${TMP[@]}")

# ---- patch scripts
source "$RUNNER_DIR/helpers/execute_patches.sh"
execute_patches "${PATCHES[@]:-}"

# ---- build the command
cd "$PRIMUS_ROOT"
export PYTHONPATH="$PRIMUS_ROOT${PYTHONPATH:+:$PYTHONPATH}"
if [[ "$SINGLE" == "1" ]]; then
  CMD=(python3 "$SCRIPT" "${PRIMUS_ARGS[@]}")
else
  CMD=(torchrun --nproc_per_node "$GPUS_PER_NODE" --nnodes "$NNODES" --node_rank "$NODE_RANK"
       --master_addr "$MASTER_ADDR" --master_port "$MASTER_PORT")
  if [[ "${PRIMUS_LOCAL_RANKS_FILTER:-}" != "" ]]; then CMD+=(--local-ranks-filter "$PRIMUS_LOCAL_RANKS_FILTER"); fi
  use_numa=0
  if [[ "$NUMA" == "on" ]] || { [[ "$NUMA" == "auto" ]] && command -v numactl >/dev/null 2>&1; }; then use_numa=1; fi
  if [[ "$use_numa" == "1" ]]; then
    CMD+=(--no-python "$RUNNER_DIR/helpers/numa_bind.sh" python3 "$SCRIPT" "${PRIMUS_ARGS[@]}")
  else
    CMD+=("$SCRIPT" "${PRIMUS_ARGS[@]}")
  fi
fi

LOG_INFO_RANK0 "launch: nodes=$NNODES node_rank=$NODE_RANK gpus_per_node=$GPUS_PER_NODE master=$MASTER_ADDR:$MASTER_PORT"
if [[ "${PRIMUS_DRY_RUN:-0}" == "1" ]]; then
  echo "[dry-run] $(quote_cmd "${CMD[@]}")"
  [[ -n "$LOG_FILE" ]] && echo "[dry-run] log file: $LOG_FILE"
  exit 0
fi

set +e
if [[ -n "$LOG_FILE" ]]; then
  mkdir -p "$(dirname "$LOG_FILE")"
  "${CMD[@]}" 2>&1 | tee "$LOG_FILE"
  rc=${PIPESTATUS[0]}
else
  "${CMD[@]}"
  rc=$?
fi
set -e
if (( rc > 128 )); then
  LOG_ERROR "worker terminated by signal $(( rc - 128 ))"
elif (( rc != 0 )); then
  LOG_ERROR "worker exited with code $rc"
else
  LOG_INFO_RANK0 "worker finished successfully"
fi
exit "$rc"
