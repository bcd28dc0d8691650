#!/usr/bin/env bash
# Builds the turbo_dllm_b200 wheel with its sm_100a kernel library inside.
#
#   packaging/build_cuda_wheels.sh [--arch 10.0a] [--out dist]
#
# Only compute capability 10.0a (B200) is accepted: the kernels use tcgen05 / TMEM / TMA instructions that
# exist on no other architecture, so a request for another one is an error, not a silent fallback.
# Counterpart of the reference's scripts/build/build_cuda_wheels.sh (which accepts 8.0, 8.9 and 9.0).
set -euo pipefail

ARCH="10.0a"
OUT="dist"
while [[ $# -gt 0 ]]; do
  case "$1" in
    --arch) ARCH="$2"; shift 2 ;;
    --out) OUT="$2"; shift 2 ;;
    -h|--help) sed -n '2,10p' "$0"; exit 0 ;;
    *) echo "unknown argument: $1" >&2; exit 2 ;;
  esac
done
if [[ "$ARCH" != "10.0a" ]]; then
  echo "error: unsupported architecture '$ARCH' (this package builds for 10.0a / sm_100a only)" >&2
  exit 2
fi
ROOT="$(cd "$(dirname "$0")/.." && pwd)"
cd "$ROOT"
command -v nvcc >/dev/null || { echo "error: nvcc not on PATH" >&2; exit 2; }
python -m turbo_dllm_b200.kernels.build --force
python -m turbo_dllm_b200.profiling.release_gates
python -m pip wheel --no-deps --no-build-isolation --wheel-dir "$OUT" .
python -m turbo_dllm_b200.profiling.portable_artifacts --kind gpu "$OUT"/turbo_dllm_b200-*.whl
echo "wheel(s) in $OUT:"
ls -l "$OUT"
