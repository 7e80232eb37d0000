"""Prompt framing and tokenisers: DeepSeek-V4 chat + DSML tool calls, GLM and MiniMax chat
framing, byte-level BPE built from GGUF metadata."""
