#!/usr/bin/env bash
# primus-cli slurm: run through Slurm.
#
#   primus-cli slurm [srun|sbatch] [slurm flags ...] -- [container|direct] [mode args] -- <primus args>
#
# Every flag before the first `--` goes to srun / sbatch unchanged (e.g. -N 4 -p gpu --time 2:00:00).
# One task per node runs runner/primus-cli-slurm-entry.sh, which exports NODE_RANK / NNODES /
# MASTER_ADDR from Slurm's variables and then starts the requested mode on that node.
set -euo pipefail
RUNNER_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
export PRIMUS_ROOT="${PRIMUS_ROOT:-$(cd "$RUNNER_DIR/.." && pwd)}"
source "$RUNNER_DIR/lib/common.sh"
source "$RUNNER_DIR/lib/config.sh"
source "$RUNNER_DIR/lib/validation.sh"
load_config_auto "$RUNNER_DIR" "${PRIMUS_CLI_CONFIG_FILE:-}" || exit 2

LAUNCHER="$(cfg_get slurm.launcher srun)"
case "${1:-}" in srun|sbatch) LAUNCHER="$1"; shift ;; esac
SLURM_FLAGS=()
while [[ $# -gt 0 ]]; do
  case "$1" in
    --) shift; break ;;
    -h|--help) sed -n '2,9p' "${BASH_SOURCE[0]}" | sed 's/^# \{0,1\}//'; exit 0 ;;
    *) SLURM_FLAGS+=("$1"); shift ;;
  esac
done
[[ $# -gt 0 ]] || usage_error "nothing to run (expected: -- direct -- train pretrain ...)"
ENTRY_ARGS=("$@")
case "${ENTRY_ARGS[0]}" in container|direct) ;; *) ENTRY_ARGS=(direct -- "${ENTRY_ARGS[@]}") ;; esac

# defaults from the config file unless given on the command line
has_flag() { local f; for f in "${SLURM_FLAGS[@]:-}"; do [[ "$f" == "$1" || "$f" == "$1="* || "$f" == "$2" ]] && return 0; done; return 1; }
has_flag --nodes -N || SLURM_FLAGS+=(--nodes "$(cfg_get slurm.nodes 1)")
p="$(cfg_get slurm.partition "")"; [[ -n "$p" ]] && ! has_flag --partition -p && SLURM_FLAGS+=(--partition "$p")
t="$(cfg_get slurm.time "")"; [[ -n "$t" ]] && ! has_flag --time -t && SLURM_FLAGS+=(--time "$t")
has_flag --ntasks-per-node --ntasks-per-node || SLURM_FLAGS+=(--ntasks-per-node 1)

[[ "${PRIMUS_DRY_RUN:-0}" == "1" ]] || require_cmd "$LAUNCHER"
CMD=("$LAUNCHER" "${SLURM_FLAGS[@]}")
if [[ "$LAUNCHER" == "sbatch" ]]; then
  CMD+=(--wrap "srun bash $(printf '%q' "$RUNNER_DIR/primus-cli-slurm-entry.sh") $(quote_cmd "${ENTRY_ARGS[@]}")")
else
  CMD+=(bash "$RUNNER_DIR/primus-cli-slurm-entry.sh" "${ENTRY_ARGS[@]}")
fi
if [[ "${PRIMUS_DRY_RUN:-0}" == "1" ]]; then echo "[dry-run] $(quote_cmd "${CMD[@]}")"; exit 0; fi
exec "${CMD[@]}"
