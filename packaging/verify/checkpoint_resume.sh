#!/usr/bin/env bash
# Save after a step, reload, continue: the result must equal the uninterrupted run bit for bit.
set -euo pipefail
cd "$(cd "$(dirname "$0")/../.." && pwd)"
python -m pytest tests -x -q -m checkpoint_resume
