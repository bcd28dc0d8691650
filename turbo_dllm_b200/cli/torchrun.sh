#!/usr/bin/env bash
# Thin wrapper: one node (or one node of several) through `dllm launch`.
#   NPROC=8 ./torchrun.sh --config train.yaml [dllm launch flags...]
# Counterpart of the reference's scripts/launch/torchrun.sh.
set -euo pipefail
exec python -m turbo_dllm_b200.cli.main launch --nproc-per-node "${NPROC:-8}" \
  --master-addr "${MASTER_ADDR:-127.0.0.1}" --master-port "${MASTER_PORT:-29500}" "$@"
