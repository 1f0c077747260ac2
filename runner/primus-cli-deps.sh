#!/usr/bin/env bash
# primus-cli deps: optional third-party checkouts pinned in runner/_thirdparty.lock
#   primus-cli deps sync [--dir DIR]      clone / update every pinned repository
#   primus-cli deps list                  print the pins
# This framework has no mandatory third-party source dependency (single native backend); the lock file
# lists optional tools such as tokenizer assets or evaluation harnesses.
set -euo pipefail
RUNNER_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
source "$RUNNER_DIR/lib/common.sh"
LOCK="$RUNNER_DIR/_thirdparty.lock"
ACTION="${1:-}"; shift || true
DIR="${PRIMUS_ROOT:-$RUNNER_DIR/..}/third_party"
while [[ $# -gt 0 ]]; do case "$1" in --dir) DIR="$2"; shift 2 ;; *) usage_error "unknown deps option $1" ;; esac; done
case "$ACTION" in
  list) [[ -f "$LOCK" ]] && grep -v '^#' "$LOCK" || true ;;
  sync)
    [[ -f "$LOCK" ]] || { LOG_INFO "no lock file: nothing to sync"; exit 0; }
    mkdir -p "$DIR"
    while read -r name url rev; do
      [[ -z "$name" || "$name" == \#* ]] && continue
      if [[ -d "$DIR/$name/.git" ]]; then
        run_or_print git -C "$DIR/$name" fetch --quiet origin
      else
        run_or_print git clone --quiet "$url" "$DIR/$name"
      fi
      run_or_print git -C "$DIR/$name" checkout --quiet "$rev"
    done < "$LOCK" ;;
  *) usage_error "usage: primus-cli deps {sync [--dir DIR] | list}" ;;
esac
