#!/usr/bin/env bash
# Launcher configuration: `.primus.yaml` (system file next to the launcher, then ~/.primus.yaml, then the
# file given with --config) flattened into the associative array PRIMUS_CFG with keys "section.key" or
# "section.sub.key".  Only the YAML subset the defaults file uses is understood: nested mappings by
# two-space indentation, scalars, and "- item" lists (joined with newlines).
# Precedence when the scripts read a value: command line > user file > system file.

declare -gA PRIMUS_CFG

_cfg_trim() { local s="$1"; s="${s#"${s%%[![:space:]]*}"}"; s="${s%"${s##*[![:space:]]}"}"; s="${s%\"}"; s="${s#\"}"; s="${s%\'}"; s="${s#\'}"; printf '%s' "$s"; }

load_config_file() {
  local file="$1"
  [[ -f "$file" ]] || return 0
  local -a stack=()
  local line key val indent depth last_key=""
  while IFS= read -r line || [[ -n "$line" ]]; do
    [[ "$line" =~ ^[[:space:]]*# ]] && continue
    [[ "$line" =~ ^[[:space:]]*$ ]] && continue
    line="${line%%[[:space:]]#*}"
    indent="${line%%[![:space:]]*}"
    depth=$(( ${#indent} / 2 ))
    local body="${line#"$indent"}"
    if [[ "$body" == "- "* ]]; then
      val="$(_cfg_trim "${body#- }")"
      local full
      full="$(IFS=.; echo "${stack[*]:0:$depth}")"
      if [[ -n "${PRIMUS_CFG[$full]:-}" ]]; then PRIMUS_CFG[$full]+=$'\n'"$val"; else PRIMUS_CFG[$full]="$val"; fi
      continue
    fi
    key="$(_cfg_trim "${body%%:*}")"
    val="$(_cfg_trim "${body#*:}")"
    stack=("${stack[@]:0:$depth}")
    stack[$depth]="$key"
    if [[ -n "$val" ]]; then
      local full
      full="$(IFS=.; echo "${stack[*]:0:$((depth + 1))}")"
      PRIMUS_CFG[$full]="$val"
    else
      local full
      full="$(IFS=.; echo "${stack[*]:0:$((depth + 1))}")"
      unset "PRIMUS_CFG[$full]"
    fi
  done < "$file"
}

load_config_auto() {
  local runner_dir="$1" explicit="${2:-}"
  load_config_file "$runner_dir/.primus.yaml"
  load_config_file "${HOME:-/root}/.primus.yaml"
  [[ -n "$explicit" ]] && { [[ -f "$explicit" ]] || { echo "config file $explicit not found" >&2; return 2; }; load_config_file "$explicit"; }
  return 0
}

cfg_get() { local k="$1" d="${2:-}"; if [[ -n "${PRIMUS_CFG[$k]+x}" ]]; then printf '%s' "${PRIMUS_CFG[$k]}"; else printf '%s' "$d"; fi; }

# names of the keys directly below a section, e.g. extract_config_section container.options
extract_config_section() {
  local prefix="$1." k
  for k in "${!PRIMUS_CFG[@]}"; do
    [[ "$k" == "$prefix"* ]] && echo "${k#"$prefix"}"
  done | sort
}
