#!/usr/bin/env bash
# Raw-block GGUF generation on N GPUs of one node (experts split over the ranks, one process per GPU).
#   GGUF=/models/MiniMax-M2.gguf NPROC=8 TOKENS=1,2,3,4 MAX_NEW=64 ./run_generate_gguf_tp.sh [extra generate_gguf flags]
# Extra flags go to every rank, e.g. --gpu-memory-gib 160 (experts beyond the budget are staged from pinned host memory),
# --layers 8, --prewarm. A seed file of raw int32 / int64 token ids can replace TOKENS: SEED_FILE=/path/ids.bin.
set -euo pipefail
: "${GGUF:?set GGUF to a .gguf file (or the first shard of a split file)}"
NPROC="${NPROC:-8}"
PROMPT_ARGS=(--tokens "${TOKENS:-1,2,3,4,5,6,7,8}")
if [[ -n "${SEED_FILE:-}" ]]; then PROMPT_ARGS=(--seed-file "$SEED_FILE"); fi
if [[ "$NPROC" == "1" ]]; then
  exec python -m pocketllm_b200.cli.generate_gguf --gguf-path "$GGUF" "${PROMPT_ARGS[@]}" --max-new-tokens "${MAX_NEW:-32}" \
    --max-context "${MAX_CONTEXT:-4096}" "$@"
fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NPROC" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29531}" \
  -m pocketllm_b200.cli.generate_gguf --gguf-path "$GGUF" "${PROMPT_ARGS[@]}" --max-new-tokens "${MAX_NEW:-32}" \
  --max-context "${MAX_CONTEXT:-4096}" "$@"
