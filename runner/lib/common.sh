#!/usr/bin/env bash
# Shared helpers of the launcher scripts: logging, errors, small utilities.
# Exit codes: 0 ok, 1 generic failure, 2 usage error, 3 missing dependency / environment problem.

: "${PRIMUS_LOG_LEVEL:=INFO}"

_primus_ts() { date '+%Y-%m-%d %H:%M:%S'; }
_primus_rank() { echo "${NODE_RANK:-${SLURM_NODEID:-0}}"; }

LOG_DEBUG() { [[ "${PRIMUS_LOG_LEVEL}" == "DEBUG" ]] && echo "[$(_primus_ts)][node-$(_primus_rank)][DEBUG] $*" >&2; return 0; }
LOG_INFO() { [[ "${PRIMUS_SILENT:-0}" == "1" ]] || echo "[$(_primus_ts)][node-$(_primus_rank)][INFO] $*" >&2; }
LOG_WARN() { echo "[$(_primus_ts)][node-$(_primus_rank)][WARN] $*" >&2; }
LOG_ERROR() { echo "[$(_primus_ts)][node-$(_primus_rank)][ERROR] $*" >&2; }
LOG_INFO_RANK0() { [[ "$(_primus_rank)" == "0" ]] && LOG_INFO "$@"; return 0; }

die() { LOG_ERROR "$1"; exit "${2:-1}"; }
usage_error() { LOG_ERROR "$1"; exit 2; }
require_cmd() { command -v "$1" >/dev/null 2>&1 || die "required command '$1' not found" 3; }

# print a command line with shell quoting, one token per argument
quote_cmd() { local out=""; local a; for a in "$@"; do out+="$(printf '%q' "$a") "; done; echo "${out% }"; }

# run or, with PRIMUS_DRY_RUN=1, only print
run_or_print() {
  if [[ "${PRIMUS_DRY_RUN:-0}" == "1" ]]; then
    echo "[dry-run] $(quote_cmd "$@")"
  else
    "$@"
  fi
}
