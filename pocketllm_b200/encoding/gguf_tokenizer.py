"""Byte-level BPE tokenizer assembled from GGUF metadata (`tokenizer.ggml.tokens`,
`.merges`, `.token_type`, `.pre`), on the Hugging Face `tokenizers` runtime.

`tokenizer.ggml.pre` values of the llama3 / GLM-4 family need the regex split (contractions,
words, 1-3 digit groups, punctuation runs, newline and whitespace runs) before the
byte-level step; every other value keeps plain ByteLevel
(reference: src/encoding/gguf_tokenizer.py:9-60).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Iterable

from ..formats import gguf

LLAMA3_STYLE_PRE = frozenset({"glm4", "chatglm-bpe", "llama3", "llama-bpe", "llama-v3", "llama3-bpe"})
LLAMA3_SPLIT = (r"(?:'[sS]|'[tT]|'[rR][eE]|'[vV][eE]|'[mM]|'[lL][lL]|'[dD])|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}"
                r"| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
TOKEN_TYPE_CONTROL, TOKEN_TYPE_USER_DEFINED = 3, 4


def read_metadata(path: str | Path) -> dict[str, Any]:
    f = gguf.GGUFFile(gguf.shard_paths(path)[0])
    md = dict(f.metadata)
    f.close()
    return md


def build_tokenizer(metadata: dict[str, Any]):
    """Returns a `tokenizers.Tokenizer`."""
    from tokenizers import AddedToken, Regex, Tokenizer, decoders, models, pre_tokenizers
    tokens = metadata.get("tokenizer.ggml.tokens")
    if not tokens:
        raise ValueError("GGUF metadata has no tokenizer.ggml.tokens")
    if metadata.get("tokenizer.ggml.model", "gpt2") not in ("gpt2", "bpe"):
        raise ValueError(f"unsupported tokenizer model {metadata.get('tokenizer.ggml.model')!r}")
    vocab = {t: i for i, t in enumerate(tokens)}
    merges = []
    for m in metadata.get("tokenizer.ggml.merges", []):
        a, _, b = m.partition(" ")
        if a in vocab and b in vocab:
            merges.append((a, b))
    tok = Tokenizer(models.BPE(vocab=vocab, merges=merges, fuse_unk=False, byte_fallback=False))
    pre = metadata.get("tokenizer.ggml.pre")
    if pre and str(pre) in LLAMA3_STYLE_PRE:
        tok.pre_tokenizer = pre_tokenizers.Sequence([
            pre_tokenizers.Split(Regex(LLAMA3_SPLIT), behavior="isolated", invert=False),
            pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    else:
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    types = metadata.get("tokenizer.ggml.token_type", [])
    special = [AddedToken(tokens[i], special=True, normalized=False) for i, t in enumerate(types)
               if t in (TOKEN_TYPE_CONTROL, TOKEN_TYPE_USER_DEFINED) and i < len(tokens)]
    if special:
        tok.add_special_tokens(special)
    return tok


def context_length(metadata: dict[str, Any], default: int = 4096) -> int:
    arch = metadata.get("general.architecture", "")
    return int(metadata.get(f"{arch}.context_length", default))


def special_ids(metadata: dict[str, Any]) -> dict[str, int | None]:
    g = lambda k: (int(metadata[k]) if k in metadata else None)
    return {"bos": g("tokenizer.ggml.bos_token_id"), "eos": g("tokenizer.ggml.eos_token_id"),
            "pad": g("tokenizer.ggml.padding_token_id"), "eot": g("tokenizer.ggml.eot_token_id")}


def parse_ids_csv(text: str) -> list[int]:
    return [int(t) for t in text.replace("\n", ",").split(",") if t.strip()]


def decode_ids(tok, ids: Iterable[int], skip_special: bool = False) -> str:
    return tok.decode([int(i) for i in ids], skip_special_tokens=skip_special)
