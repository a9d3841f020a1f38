#!/usr/bin/env bash
# Environment -> flags for examples/serve_sessions.py (one process per GPU through torchrun).
set -euo pipefail
cd "$(dirname "$0")/.."
GPUS="${NAIVERT_GPUS:-8}"
ARGS=(--host "${NAIVERT_HOST:-0.0.0.0}" --port "${NAIVERT_PORT:-8080}" --model "${NAIVERT_MODEL:-naive-n0.5}")
[[ -n "${NAIVERT_TARGET_CHECKPOINT:-}" ]] && ARGS+=(--target "$NAIVERT_TARGET_CHECKPOINT")
[[ -n "${NAIVERT_DRAFT_CHECKPOINT:-}" ]] && ARGS+=(--draft "$NAIVERT_DRAFT_CHECKPOINT")
[[ "${NAIVERT_RANDOM_INIT:-0}" == "1" ]] && ARGS+=(--random-init)
[[ -n "${NAIVERT_LAYERS:-}" ]] && ARGS+=(--layers "$NAIVERT_LAYERS")
[[ -n "${NAIVERT_SERVED_MODEL_NAME:-}" ]] && ARGS+=(--served-model-name "$NAIVERT_SERVED_MODEL_NAME")
[[ -n "${NAIVERT_CAPACITY:-}" ]] && ARGS+=(--capacity "$NAIVERT_CAPACITY")
[[ -n "${NAIVERT_MAX_DECODE_TOKENS:-}" ]] && ARGS+=(--max-decode-tokens "$NAIVERT_MAX_DECODE_TOKENS")
[[ -n "${NAIVERT_OUTPUT_CAPACITY:-}" ]] && ARGS+=(--output-capacity "$NAIVERT_OUTPUT_CAPACITY")
[[ -n "${NAIVERT_STORE_GB:-}" ]] && ARGS+=(--store-gb "$NAIVERT_STORE_GB")
[[ -n "${NAIVERT_QUEUE_DEPTH:-}" ]] && ARGS+=(--queue-depth "$NAIVERT_QUEUE_DEPTH")
[[ -n "${NAIVERT_SEED:-}" ]] && ARGS+=(--seed "$NAIVERT_SEED")
[[ -n "${NAIVERT_TEMPERATURE:-}" ]] && ARGS+=(--temperature "$NAIVERT_TEMPERATURE")
[[ -n "${NAIVERT_TOP_P:-}" ]] && ARGS+=(--top-p "$NAIVERT_TOP_P")
[[ -n "${NAIVERT_CORS_ORIGIN:-}" ]] && ARGS+=(--cors-origin "$NAIVERT_CORS_ORIGIN")
[[ -n "${NAIVERT_RESUME_POLICY:-}" ]] && ARGS+=(--resume-policy "$NAIVERT_RESUME_POLICY")
[[ -n "${NAIVERT_PREFILL:-}" ]] && ARGS+=(--prefill "$NAIVERT_PREFILL")
[[ -n "${NAIVERT_PREFILL_CHUNK:-}" ]] && ARGS+=(--prefill-chunk "$NAIVERT_PREFILL_CHUNK")
if [[ "${NAIVERT_DRY_RUN:-0}" == "1" ]]; then
  echo "gpus=$GPUS" "${ARGS[@]}"
  exit 0
fi
if [[ "$GPUS" -gt 1 ]]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 \
       examples/serve_sessions.py "${ARGS[@]}" "$@"
fi
exec python examples/serve_sessions.py "${ARGS[@]}" "$@"
