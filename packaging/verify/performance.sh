#!/usr/bin/env bash
# Performance tier: records throughput figures (JSON lines), encodes no hardware baseline.
set -euo pipefail
cd "$(cd "$(dirname "$0")/../.." && pwd)"
python -m pytest tests -x -q -m "performance and gpu" -s
python -m turbo_dllm_b200.benchmarks.gemm_bench --shapes 8192x8192x8192 --layouts kk --iters 5
