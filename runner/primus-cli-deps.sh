#!/usr/bin/env bash
# primus-cli deps: optional third-party checkouts pinned in runner/_thirdparty.lock
#   primus-cli deps sync [--dir DIR]      clone / update every pinned repository
#   primus-cli deps list                  print the pins
#   primus-cli deps check                 toolchain and Python packages the framework needs, and the state of the
#                                         native library (built? older than its sources?)
#   primus-cli deps build                 (re)build the native library (nvcc, sm_100a)
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
  check)
    rc=0
    for tool in python3 nvcc git; do
      if command -v "$tool" >/dev/null 2>&1; then echo "ok       $tool: $(command -v "$tool")"; else echo "MISSING  $tool"; rc=1; fi
    done
    python3 - <<'PY' || rc=1
import importlib, sys
need = {"torch": "2.4", "numpy": "1.24", "yaml": None, "tabulate": None}
bad = 0
for mod, minimum in need.items():
    try:
        m = importlib.import_module(mod)
        v = getattr(m, "__version__", "?")
        low = minimum is not None and tuple(int(x) for x in v.split("+")[0].split(".")[:2]) < tuple(int(x) for x in minimum.split("."))
        print(("TOO OLD " if low else "ok      ") + f" {mod} {v}" + (f" (need >= {minimum})" if low else ""))
        bad += low
    except Exception as e:
        print(f"MISSING  {mod}: {e}")
        bad += 1
for mod in ("transformers", "sentencepiece", "tensorboard", "mlflow", "wandb"):
    try:
        importlib.import_module(mod)
        print(f"ok       {mod} (optional)")
    except Exception:
        print(f"absent   {mod} (optional)")
sys.exit(1 if bad else 0)
PY
    LIB="${PRIMUS_ROOT:-$RUNNER_DIR/..}/primus_b200/lib/libprimus_b200.so"
    SRC="${PRIMUS_ROOT:-$RUNNER_DIR/..}/primus_b200/csrc"
    if [[ ! -f "$LIB" ]]; then echo "MISSING  native library $LIB (primus-cli deps build)"; rc=1
    elif [[ -n "$(find "$SRC" -newer "$LIB" \( -name '*.cu' -o -name '*.cuh' -o -name '*.h' \) -print -quit)" ]]; then
      echo "STALE    native library is older than its sources (primus-cli deps build)"; rc=1
    else echo "ok       native library $LIB"; fi
    exit $rc ;;
  build) run_or_print python3 -m primus_b200.build ;;
  *) usage_error "usage: primus-cli deps {sync [--dir DIR] | list | check | build}" ;;
esac
