#!/usr/bin/env bash
# Python OpenAI-compatible server (single process, or several ranks under torchrun for the tensor-parallel engines).
#   CKPT=/path/to/ckpt PORT=8000 ./run_openai_server.sh                  # backend detected from the checkpoint (MODEL=qwen|gguf|dsv4 forces it)
#   CKPT=/path/to/ckpt GPUS=4 ./run_openai_server.sh                     # rank 0 serves, the other ranks follow its requests
#   SERVING_PROFILE=safe1|latency2|throughput4 picks a profile of the typed configuration; CONFIG=file.json|yaml adds a file;
#   PARTITION_POLICY=layer_pp runs DeepSeek-V4 as a layer pipeline over the ranks instead of expert parallelism.
set -euo pipefail
: "${CKPT:?set CKPT to a checkpoint directory or GGUF file}"
ARGS=(--ckpt "$CKPT" --host "${HOST:-127.0.0.1}" --port "${PORT:-8000}" --max-context "${MAX_CONTEXT:-8192}")
if [ -n "${MODEL:-}" ]; then ARGS+=(--model "$MODEL"); fi
if [ -n "${CONFIG:-}" ]; then ARGS+=(--config "$CONFIG"); fi
if [ -n "${TOKENIZER_PATH:-}" ]; then ARGS+=(--tokenizer-path "$TOKENIZER_PATH"); fi
if [ "${GPUS:-1}" -gt 1 ]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29555}" \
    -m pocketllm_b200.server.openai "${ARGS[@]}" "$@"
fi
exec python -m pocketllm_b200.server.openai "${ARGS[@]}" "$@"
