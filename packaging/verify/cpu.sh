#!/usr/bin/env bash
# CPU install check: the package imports, prints what it supports, validates every packaged recipe,
# byte-compiles, and passes the release gates. Needs no GPU.
set -euo pipefail
ROOT="$(cd "$(dirname "$0")/../.." && pwd)"
cd "$ROOT"
python -m turbo_dllm_b200.training --print-supported-configs > /dev/null
python - <<'PY'
from turbo_dllm_b200.config.run_spec import load_run_spec
from turbo_dllm_b200.recipes import list_recipes, recipe_path
for r in list_recipes():
    load_run_spec(recipe_path(r["name"])).validate()
    print("valid:", r["name"])
PY
python -m compileall -q turbo_dllm_b200 bench.py __graft_entry__.py
python -m turbo_dllm_b200.profiling.release_gates > /dev/null
python -m turbo_dllm_b200.cli.main launch --recipe cpu-config --nproc-per-node 2 --dry-run > /dev/null
echo "cpu install check passed"
