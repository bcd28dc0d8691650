#!/usr/bin/env bash
# End-to-end check of an exported DFlash2 drafter behind a speculative-decoding server (vLLM or SGLang, installed
# separately): validate the export, start the server, wait until it answers, gate on one greedy completion.
#   packaging/verify/serving_dflash2.sh vllm|sglang TARGET_MODEL EXPORT_DIR BLOCK_SIZE PROMPT EXPECTED_TEXT_FILE
set -euo pipefail
BACKEND="$1"; TARGET="$2"; EXPORT="$3"; BLOCK="$4"; PROMPT="$5"; EXPECTED="$6"
cd "$(cd "$(dirname "$0")/../.." && pwd)"
PORT=$([[ "$BACKEND" == vllm ]] && echo 8000 || echo 30000)
python -m turbo_dllm_b200.cli.main dflash validate-export "$EXPORT" --block-size "$BLOCK"
[[ "$BACKEND" == vllm ]] && python -m turbo_dllm_b200.cli.main dflash validate-vllm "$EXPORT" --block-size "$BLOCK"
python -m turbo_dllm_b200.cli.main dflash "serve-$BACKEND" --target-model "$TARGET" --draft "$EXPORT" \
    --block-size "$BLOCK" --port "$PORT" --launch --log "serve-$BACKEND.log" &
SERVER=$!
trap 'kill "$SERVER" 2>/dev/null || true' EXIT
for _ in $(seq 1 360); do
  curl -sf "http://127.0.0.1:$PORT/v1/models" > /dev/null && break
  kill -0 "$SERVER" 2>/dev/null || { echo "server exited; see serve-$BACKEND.log" >&2; exit 1; }
  sleep 5
done
python -m turbo_dllm_b200.cli.main dflash "verify-$BACKEND" --base-url "http://127.0.0.1:$PORT" --model "$TARGET" \
    --prompt "$PROMPT" --expected-text "$(cat "$EXPECTED")" --block-size "$BLOCK"
