#!/usr/bin/env bash
# Python OpenAI-compatible server (single process, or several ranks under torchrun for the tensor-parallel engines).
#   MODEL=qwen CKPT=/path/to/ckpt PORT=8000 ./run_openai_server.sh
#   MODEL=qwen CKPT=/path/to/ckpt GPUS=4 ./run_openai_server.sh      # rank 0 serves, the other ranks follow its requests
set -euo pipefail
: "${CKPT:?set CKPT to a checkpoint directory or GGUF file}"
ARGS=(--model "${MODEL:-qwen}" --ckpt "$CKPT" --host "${HOST:-127.0.0.1}" --port "${PORT:-8000}" --max-context "${MAX_CONTEXT:-8192}")
if [ "${GPUS:-1}" -gt 1 ]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29555}" \
    -m pocketllm_b200.server.openai "${ARGS[@]}" "$@"
fi
exec python -m pocketllm_b200.server.openai "${ARGS[@]}" "$@"
