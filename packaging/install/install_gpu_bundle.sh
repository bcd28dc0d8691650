#!/usr/bin/env bash
# Installs the prebuilt kernel bundle that matches this interpreter, CUDA runtime and GPU from a bundle catalog
# (a URL or a local file), after checking the machine.
#   packaging/install/install_gpu_bundle.sh CATALOG [--dry-run]
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
"$HERE/check_system_requirements.sh"
python -m turbo_dllm_b200.kernels.bundle_manifest install "$1" "${@:2}"
