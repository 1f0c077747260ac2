#!/usr/bin/env bash
# Runs the shell patch scripts given with --patch, in order, before the launch.
execute_patches() {
  local p
  for p in "$@"; do
    [[ -z "$p" ]] && continue
    [[ -f "$p" ]] || p="$RUNNER_DIR/helpers/patches/$p"
    [[ -f "$p" ]] || die "patch script $p not found" 2
    LOG_INFO_RANK0 "patch: $p"
    if [[ "${PRIMUS_DRY_RUN:-0}" == "1" ]]; then echo "[dry-run] bash $p"; else bash "$p" || die "patch $p failed" 1; fi
  done
}
