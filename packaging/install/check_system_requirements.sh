#!/usr/bin/env bash
# What the sm_100a build needs on a machine: a Blackwell GPU (compute capability 10.0), a driver for CUDA >= 12.8,
# Python 3.10+, and (for building from source) nvcc >= 12.8. Reads settings only; changes nothing.
set -uo pipefail
fail=0
say() { printf '%-28s %s\n' "$1" "$2"; }
py=$(python3 -c 'import sys; print("%d.%d" % sys.version_info[:2])' 2>/dev/null || echo none)
say "python" "$py"
python3 -c 'import sys; sys.exit(0 if sys.version_info >= (3, 10) else 1)' 2>/dev/null || { say "" "need Python >= 3.10"; fail=1; }
if command -v nvidia-smi > /dev/null; then
  while IFS=, read -r name cap drv; do
    say "gpu" "$name (compute $cap, driver $drv)"
    [[ "${cap// /}" == 10.* ]] || { say "" "this GPU is not sm_100: the kernel library will not load on it"; fail=1; }
  done < <(nvidia-smi --query-gpu=name,compute_cap,driver_version --format=csv,noheader)
else
  say "gpu" "nvidia-smi not found (CPU-only use: configuration, data preparation, planning)"
fi
if command -v nvcc > /dev/null; then
  ver=$(nvcc --version | sed -n 's/.*release \([0-9]*\.[0-9]*\).*/\1/p')
  say "nvcc" "$ver"
  python3 - "$ver" <<'PY' || { say "" "building the kernels needs nvcc >= 12.8 (sm_100a)"; fail=1; }
import sys
major, minor = (int(x) for x in sys.argv[1].split("."))
sys.exit(0 if (major, minor) >= (12, 8) else 1)
PY
else
  say "nvcc" "not found (only needed to build the kernel library from source)"
fi
python3 -c 'import torch; print("%-28s %s (cuda %s)" % ("torch", torch.__version__, torch.version.cuda))' 2>/dev/null \
  || { say "torch" "not importable"; fail=1; }
exit $fail
