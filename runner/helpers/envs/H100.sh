#!/usr/bin/env bash
# Listed for completeness: the kernels of this framework target sm_100a only.
echo "[primus-env] H100 detected: primus_b200 kernels require a B200 (sm_100a)" >&2
