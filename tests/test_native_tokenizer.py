"""Native byte-level BPE tokenizer against the `tokenizers` library on a vocabulary trained in the test."""
import ctypes
import json
import subprocess
from pathlib import Path

import pytest

from pocketllm_b200.encoding import gguf_tokenizer
from pocketllm_b200.formats import gguf

ROOT = Path(__file__).resolve().parent.parent
CORPUS = ["The quick brown fox jumps over the lazy dog.", "It's 2024, isn't it? We've seen 1,234 things; they'll see more!",
          "def f(x):\n    return x * 2  # twice\n\n", "Tabs\tand  double  spaces   and trailing   ", "naïve café über straße",
          "hello world hello there general kenobi", "I'd say you're right, she's 42 and he'll be 7."] * 3
TEXTS = ["Hello, world! It's me.", "  leading spaces and\ttabs\n\nnewlines  ", "x=1+2;y=[3,4]", "they'll we've I'm he'd don't 'quoted'",
         "naïve café", "a", "", "   ", "end with space ", "12345 67 8", "mixed123abc!!!", "<|eos|>after special<|eos|>", "line1\nline2\r\n  indented"]


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    from tokenizers import Tokenizer, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.train_from_iterator(CORPUS, trainers.BpeTrainer(vocab_size=420, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), special_tokens=["<|eos|>"]))
    model = json.loads(tok.to_str())["model"]
    vocab = sorted(model["vocab"].items(), key=lambda kv: kv[1])
    tokens = [k for k, _ in vocab]
    merges = [m if isinstance(m, str) else " ".join(m) for m in model["merges"]]
    path = tmp_path_factory.mktemp("tok") / "tok.gguf"
    w = gguf.GGUFWriter()
    w.add_meta("general.architecture", "minimax-m2")
    w.add_meta("tokenizer.ggml.model", "gpt2")
    w.add_meta("tokenizer.ggml.tokens", tokens)
    w.add_meta("tokenizer.ggml.merges", merges)
    w.add_meta("tokenizer.ggml.token_type", [3 if t == "<|eos|>" else 1 for t in tokens])
    import numpy as np
    w.add_tensor("dummy", np.zeros(32, np.float32), "f32")
    w.write(path)
    tok.save(str(path.parent / "tokenizer.json"))
    return path, gguf_tokenizer.build_tokenizer(gguf_tokenizer.read_metadata(path))


def test_native_tokenizer_matches_library(trained):
    from pocketllm_b200.ops import lib
    path, ref = trained
    L = lib.engine()
    L.pk_tokenizer_from_gguf.restype = ctypes.c_void_p
    L.pk_tokenizer_decode.restype = ctypes.c_char_p
    h = ctypes.c_void_p(L.pk_tokenizer_from_gguf(str(path).encode()))
    assert h.value
    buf = (ctypes.c_int * 4096)()
    for text in TEXTS + CORPUS[:7]:
        n = L.pk_tokenizer_encode(h, text.encode(), 1, buf, 4096)
        got = list(buf[:n])
        want = ref.encode(text, add_special_tokens=False).ids
        assert got == want, (text, got, want)
        arr = (ctypes.c_int * n)(*got)
        assert L.pk_tokenizer_decode(h, arr, n, 0).decode() == text
    n = L.pk_tokenizer_encode(h, b"<|eos|>x", 0, buf, 4096)          # special tokens as plain text
    assert list(buf[:n]) != [ref.token_to_id("<|eos|>"), ref.token_to_id("x")]
    assert L.pk_tokenizer_decode(h, (ctypes.c_int * 2)(ref.token_to_id("<|eos|>"), ref.token_to_id("a")), 2, 1).decode() == "a"
    L.pk_tokenizer_destroy(h)


def test_native_tokenizer_from_tokenizer_json(trained):
    """The same vocabulary read from a Hugging Face tokenizer.json directory gives the same ids."""
    from pocketllm_b200.ops import lib
    path, ref = trained
    L = lib.engine()
    L.pk_tokenizer_from_hf.restype = ctypes.c_void_p
    L.pk_tokenizer_decode.restype = ctypes.c_char_p
    h = ctypes.c_void_p(L.pk_tokenizer_from_hf(str(path.parent).encode()))
    assert h.value, L.pk_engine_last_error()
    buf = (ctypes.c_int * 4096)()
    for text in TEXTS + CORPUS[:7]:
        n = L.pk_tokenizer_encode(h, text.encode(), 1, buf, 4096)
        assert list(buf[:n]) == ref.encode(text, add_special_tokens=False).ids, text
        assert L.pk_tokenizer_decode(h, (ctypes.c_int * n)(*buf[:n]), n, 0).decode() == text
    L.pk_tokenizer_destroy(h)
    assert not L.pk_tokenizer_from_hf(str(path.parent / "missing").encode())
    exe = ROOT / "pocketllm_b200" / "_C" / "pocket_engine"
    out = subprocess.run([str(exe), "--tokenizer-dir", str(path.parent), "--tokenize", "Hello, world!"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0 and [int(t) for t in out.stdout.strip().split("=", 1)[1].split(",")] == ref.encode("Hello, world!", add_special_tokens=False).ids


def test_tokenizer_cli_tool(trained):
    path, ref = trained
    exe = ROOT / "pocketllm_b200" / "_C" / "pocket_engine"
    out = subprocess.run([str(exe), "--tokenizer-gguf", str(path), "--tokenize", "Hello, world!"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    ids = [int(t) for t in out.stdout.strip().split("=", 1)[1].split(",")]
    assert ids == ref.encode("Hello, world!", add_special_tokens=False).ids
    out = subprocess.run([str(exe), "--tokenizer-gguf", str(path), "--detokenize", ",".join(map(str, ids))], capture_output=True, text=True, timeout=60)
    assert out.stdout.strip() == "text=Hello, world!"
