#!/usr/bin/env bash
# Native OpenAI front end (C++ HTTP / SSE, request validation, sampler settings) in front of a Python model worker: the way
# to serve DeepSeek-V4 and the GGUF families (MiniMax-M2, GLM-DSA) from pocket_engine.
#   MODEL=dsv4 CKPT=/models/DeepSeek-V4-Flash RANKS=8 PORT=8000 ./run_native_serve_worker.sh
#   MODEL=gguf CKPT=/models/MiniMax-M2.gguf TOKENIZER=gguf:/models/MiniMax-M2.gguf CHAT_FORMAT=minimax ./run_native_serve_worker.sh
# RANKS > 1 starts the worker under torchrun (one rank per GPU; rank 0 talks to the front end, the others follow its requests).
set -euo pipefail
: "${CKPT:?set CKPT to a checkpoint directory or GGUF file}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ENGINE="${ENGINE:-$HERE/../_C/pocket_engine}"
MODEL="${MODEL:-dsv4}"
case "$MODEL" in
  dsv4) DEFAULT_TOKENIZER="hf:$CKPT"; DEFAULT_CHAT=dsv4 ;;
  qwen) DEFAULT_TOKENIZER="hf:$CKPT"; DEFAULT_CHAT=qwen ;;
  gguf) DEFAULT_TOKENIZER="gguf:$CKPT"; DEFAULT_CHAT="${CHAT_FORMAT:-glm}" ;;
  *) echo "MODEL must be dsv4, qwen or gguf" >&2; exit 1 ;;
esac
exec "$ENGINE" --serve --model-worker "$MODEL" --ckpt "$CKPT" --worker-ranks "${RANKS:-1}" --worker-master-port "${MASTER_PORT:-29641}" \
  --host "${HOST:-127.0.0.1}" --port "${PORT:-8000}" --max-context "${MAX_CONTEXT:-8192}" --model-name "${MODEL_NAME:-pocketllm-b200}" \
  --tokenizer "${TOKENIZER:-$DEFAULT_TOKENIZER}" --chat-format "${CHAT_FORMAT:-$DEFAULT_CHAT}" --sidecar-python "${PYTHON:-python}" "$@"
