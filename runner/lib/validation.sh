#!/usr/bin/env bash
# Parameter validation used by the launcher modes.

is_int() { [[ "$1" =~ ^[0-9]+$ ]]; }

validate_int_range() { # name value min max
  is_int "$2" || usage_error "$1 must be a non-negative integer (got '$2')"
  (( $2 >= $3 && $2 <= $4 )) || usage_error "$1 must be in [$3, $4] (got $2)"
}

validate_distributed_params() {
  validate_int_range GPUS_PER_NODE "${GPUS_PER_NODE}" 1 16
  validate_int_range NNODES "${NNODES}" 1 65536
  validate_int_range NODE_RANK "${NODE_RANK}" 0 $(( NNODES - 1 ))
  validate_int_range MASTER_PORT "${MASTER_PORT}" 1024 65535
  [[ -n "${MASTER_ADDR}" ]] || usage_error "MASTER_ADDR must not be empty"
  [[ "${MASTER_ADDR}" =~ ^[A-Za-z0-9._:-]+$ ]] || usage_error "MASTER_ADDR has invalid characters: ${MASTER_ADDR}"
}

validate_env_assignment() { [[ "$1" =~ ^[A-Za-z_][A-Za-z0-9_]*=.*$ ]] || usage_error "--env expects KEY=VALUE (got '$1')"; }
validate_file() { [[ -f "$1" ]] || usage_error "$2 '$1' does not exist"; }
validate_memory_format() { [[ "$1" =~ ^[0-9]+[bkmgBKMG]?$ ]] || usage_error "memory size '$1' is not of the form 64g / 512m"; }
validate_cpus_format() { [[ "$1" =~ ^[0-9]+(\.[0-9]+)?$ ]] || usage_error "cpus '$1' must be a number"; }
validate_volume_format() { [[ "$1" == *:* || "$1" == /* ]] || usage_error "volume '$1' must be HOST[:CONTAINER[:MODE]]"; }
validate_slurm_env() {
  [[ -n "${SLURM_JOB_ID:-}" ]] || LOG_WARN "SLURM_JOB_ID is not set: not inside a Slurm allocation"
}
