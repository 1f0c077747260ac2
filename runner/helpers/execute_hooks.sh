#!/usr/bin/env bash
# Hook runner.  Order: global hooks runner/helpers/hooks/*.{sh,py} (sorted), then
# runner/helpers/hooks/<group>/<name>/*.{sh,py}.  A hook receives the primus arguments and may print
#   env.KEY=VALUE      -> exported into the launcher's environment
#   extra.name=value   -> `--name value` appended to the primus arguments
# Any other output is passed through to stderr.  A failing hook aborts the launch.

execute_hooks() {
  local group="$1" name="$2"; shift 2
  local hooks_root="${PRIMUS_HOOKS_DIR:-$RUNNER_DIR/helpers/hooks}"
  local -a files=()
  local f
  for f in "$hooks_root"/*.sh "$hooks_root"/*.py; do [[ -f "$f" ]] && files+=("$f"); done
  if [[ -n "$group" && -n "$name" && -d "$hooks_root/$group/$name" ]]; then
    for f in "$hooks_root/$group/$name"/*.sh "$hooks_root/$group/$name"/*.py; do [[ -f "$f" ]] && files+=("$f"); done
  fi
  [[ ${#files[@]} -eq 0 ]] && return 0
  IFS=$'\n' files=($(printf '%s\n' "${files[@]}" | sort)); unset IFS
  for f in "${files[@]}"; do
    LOG_DEBUG "hook: $f"
    local out rc
    rc=0
    if [[ "$f" == *.py ]]; then out="$(python3 "$f" "$@")" || rc=$?; else out="$(bash "$f" "$@")" || rc=$?; fi
    (( rc == 0 )) || die "hook $f failed with code $rc" 1
    local line
    while IFS= read -r line; do
      case "$line" in
        env.*=*) line="${line#env.}"; export "${line?}"; LOG_DEBUG "hook exported ${line%%=*}" ;;
        extra.*=*) line="${line#extra.}"; HOOK_EXTRA_ARGS+=("--${line%%=*}" "${line#*=}") ;;
        "") ;;
        *) echo "$line" >&2 ;;
      esac
    done <<< "$out"
  done
}
