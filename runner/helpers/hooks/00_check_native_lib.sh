#!/usr/bin/env bash
# Global hook: make sure the native kernel library is built (cross-compiles without a GPU).
ROOT="${PRIMUS_ROOT:-$(cd "$(dirname "${BASH_SOURCE[0]}")/../../.." && pwd)}"
if [[ ! -f "$ROOT/primus_b200/lib/libprimus_b200.so" ]]; then
  if [[ "${PRIMUS_DRY_RUN:-0}" == "1" ]]; then
    echo "native library missing: would run python3 -m primus_b200.build"
  else
    (cd "$ROOT" && python3 -m primus_b200.build >/dev/null) || { echo "building the native library failed" >&2; exit 1; }
  fi
fi
echo "env.PRIMUS_B200_LIB=$ROOT/primus_b200/lib/libprimus_b200.so"
