#!/usr/bin/env bash
# primus-cli container: run the direct launcher inside a docker / podman container.
#
#   primus-cli container [--image IMG] [--runtime docker|podman] [--name N] [--volume H[:C[:M]]]...
#                        [--env K[=V]]... [--device D]... [--cap-add C]... [--user U] [--network N]
#                        [--ipc M] [--cpus N] [--memory SZ] [--shm-size SZ] [--gpus SPEC] [--clean]
#                        [any other docker flag ...] -- <direct-mode args / primus args>
#
# Every `container.options.<key>: <value>` of .primus.yaml becomes `--<key> <value>`; flags on the command
# line override them; unknown `--flag value` pairs are passed to the container runtime unchanged.  The
# repository is mounted at the same path and used as the working directory.
set -euo pipefail
RUNNER_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
export PRIMUS_ROOT="${PRIMUS_ROOT:-$(cd "$RUNNER_DIR/.." && pwd)}"
source "$RUNNER_DIR/lib/common.sh"
source "$RUNNER_DIR/lib/config.sh"
source "$RUNNER_DIR/lib/validation.sh"
load_config_auto "$RUNNER_DIR" "${PRIMUS_CLI_CONFIG_FILE:-}" || exit 2

RUNTIME="$(cfg_get container.runtime docker)"
IMAGE="$(cfg_get container.image "")"
NAME=""
CLEAN=0
declare -A OPT
for k in $(extract_config_section container.options); do OPT["$k"]="$(cfg_get "container.options.$k")"; done
MULTI=()   # repeatable flags: --volume/--env/--device/--cap-add and unknown pass-through
INNER=()

while [[ $# -gt 0 ]]; do
  case "$1" in
    --image) IMAGE="$2"; shift 2 ;;
    --runtime) RUNTIME="$2"; shift 2 ;;
    --name) NAME="$2"; shift 2 ;;
    --clean) CLEAN=1; shift ;;
    --volume|-v) validate_volume_format "$2"; MULTI+=(--volume "$2"); shift 2 ;;
    --env|-e) MULTI+=(--env "$2"); shift 2 ;;
    --device) MULTI+=(--device "$2"); shift 2 ;;
    --cap-add) MULTI+=(--cap-add "$2"); shift 2 ;;
    --memory) validate_memory_format "$2"; OPT[memory]="$2"; shift 2 ;;
    --shm-size) validate_memory_format "$2"; OPT[shm-size]="$2"; shift 2 ;;
    --cpus) validate_cpus_format "$2"; OPT[cpus]="$2"; shift 2 ;;
    --user|--network|--ipc|--gpus|--ulimit|--workdir|--hostname|--pid) OPT["${1#--}"]="$2"; shift 2 ;;
    -h|--help) sed -n '2,12p' "${BASH_SOURCE[0]}" | sed 's/^# \{0,1\}//'; exit 0 ;;
    --) shift; INNER=("$@"); break ;;
    --*=*) MULTI+=("$1"); shift ;;
    --*) if [[ $# -ge 2 && "$2" != --* ]]; then MULTI+=("$1" "$2"); shift 2; else MULTI+=("$1"); shift; fi ;;
    *) usage_error "unexpected argument for container mode: $1" ;;
  esac
done
[[ -n "$IMAGE" ]] || usage_error "no container image (use --image or container.image in .primus.yaml)"
[[ ${#INNER[@]} -gt 0 ]] || usage_error "nothing to run inside the container (expected: -- train pretrain ...)"
[[ "${PRIMUS_DRY_RUN:-0}" == "1" ]] || require_cmd "$RUNTIME"

CMD=("$RUNTIME" run --rm)
[[ -n "$NAME" ]] && CMD+=(--name "$NAME")
for k in $(printf '%s\n' "${!OPT[@]}" | sort); do CMD+=("--$k" "${OPT[$k]}"); done
# environment pass-through whitelist
while IFS= read -r v; do
  [[ -n "$v" && -n "${!v:-}" ]] && CMD+=(--env "$v=${!v}")
done <<< "$(cfg_get container.env_passthrough "")"
for v in NNODES NODE_RANK MASTER_ADDR MASTER_PORT GPUS_PER_NODE PRIMUS_DRY_RUN; do
  [[ -n "${!v:-}" ]] && CMD+=(--env "$v=${!v}")
done
CMD+=(--volume "$PRIMUS_ROOT:$PRIMUS_ROOT" --workdir "$PRIMUS_ROOT")
CMD+=("${MULTI[@]:-}")
TMP=(); for a in "${CMD[@]}"; do [[ -n "$a" ]] && TMP+=("$a"); done; CMD=("${TMP[@]}")
# inside: the direct launcher, unless the inner args already name a mode
case "${INNER[0]}" in
  direct|slurm|deps) CMD+=("$IMAGE" bash "$PRIMUS_ROOT/runner/primus-cli" "${INNER[@]}") ;;
  --*) CMD+=("$IMAGE" bash "$PRIMUS_ROOT/runner/primus-cli" direct "${INNER[@]}") ;;
  *) CMD+=("$IMAGE" bash "$PRIMUS_ROOT/runner/primus-cli" direct -- "${INNER[@]}") ;;
esac

if [[ "$CLEAN" == "1" && -n "$NAME" ]]; then run_or_print "$RUNTIME" rm -f "$NAME" || true; fi
if [[ "${PRIMUS_DRY_RUN:-0}" == "1" ]]; then echo "[dry-run] $(quote_cmd "${CMD[@]}")"; exit 0; fi
exec "${CMD[@]}"
