#!/usr/bin/env bash
# Native OpenAI server, one pocket_engine process per GPU (rank 0 listens, the others replay its commands).
#   CKPT=/path/to/Qwen-FP8 TP=4 PORT=8000 TOKENIZER=hf:/path/to/Qwen-FP8 ./run_native_serve_tp.sh [extra pocket_engine flags]
# Extra flags go to every rank unchanged, e.g. --qwen-mtp --kv-cache-dtype fp8 --qwen-snapshot-interval 4096.
set -euo pipefail
: "${CKPT:?set CKPT to a checkpoint directory}"
exec python -m pocketllm_b200.cli.serve_native --ckpt "$CKPT" --tp "${TP:-4}" --host "${HOST:-127.0.0.1}" --port "${PORT:-8000}" \
  --tokenizer "${TOKENIZER:-hf:$CKPT}" --chat-format "${CHAT_FORMAT:-qwen}" --max-context "${MAX_CONTEXT:-32768}" \
  --model-name "${MODEL_NAME:-pocketllm-b200}" "$@"
