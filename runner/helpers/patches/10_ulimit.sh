#!/usr/bin/env bash
# Launch patch (run with `--patch 10_ulimit.sh` or listed in .primus.yaml): raise the open-file and locked-memory
# limits that NCCL's IB transport and pinned host staging need; a refusal is reported, not fatal.
ulimit -n 1048576 2>/dev/null || echo "could not raise the open-file limit (now $(ulimit -n))" >&2
ulimit -l unlimited 2>/dev/null || echo "could not lift the locked-memory limit (now $(ulimit -l))" >&2
