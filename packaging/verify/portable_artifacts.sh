#!/usr/bin/env bash
# A wheel / sdist must hold the required files, no stray native binaries and no forbidden tokens.
#   packaging/verify/portable_artifacts.sh dist/*.whl
set -euo pipefail
cd "$(cd "$(dirname "$0")/../.." && pwd)"
python -m turbo_dllm_b200.profiling.portable_artifacts "$@"
