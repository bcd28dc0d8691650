#!/usr/bin/env bash
# Repository gate: source-policy gates, documentation consistency, and the portable (CPU) test tier.
set -euo pipefail
ROOT="$(cd "$(dirname "$0")/../.." && pwd)"
cd "$ROOT"
python -m turbo_dllm_b200.profiling.release_gates
python -m pytest tests/test_docs_consistency.py tests/test_config.py tests/test_parallel_plan.py tests/test_services.py -x -q
