"""The engine's host C++ (JSON, readers, sampler, checkpoint audit, rendezvous, command channel, protocol models) built with
AddressSanitizer + UndefinedBehaviorSanitizer, and the protocol model again under ThreadSanitizer."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = [ROOT / "csrc" / "tests" / "host_selftest.cpp"] + [ROOT / "csrc" / "engine" / f for f in
                                                        ("json.cpp", "gguf_reader.cpp", "safetensors.cpp", "sampler.cpp", "control_plane.cpp", "qwen_audit.cpp",
                                                         "qwen_config.cpp", "tokenizer.cpp", "weight_source.cpp", "dsv4_config.cpp")]
GXX = shutil.which("g++", path="/usr/bin") or shutil.which("g++")


def _inputs(tmp_path):
    from pocketllm_b200.models import minimax_m2, qwen_hybrid as qh
    minimax_m2.write_random_gguf(tmp_path / "m.gguf", minimax_m2.MiniMaxM2Config.tiny())
    cfg = qh.QwenHybridConfig.tiny(layers=2, hidden=128, inter=256, vocab=256)
    qh.save_checkpoint(tmp_path / "st", cfg, qh.random_checkpoint(cfg, seed=0))
    (tmp_path / "scratch").mkdir()
    return [str(tmp_path / "m.gguf"), str(tmp_path / "st"), str(tmp_path / "scratch"), str(_tokenizer_gguf(tmp_path))]


def _tokenizer_gguf(tmp_path):
    """A small byte-level BPE vocabulary trained here and stored as GGUF tokenizer metadata."""
    import json
    import numpy as np
    from tokenizers import Tokenizer, models, pre_tokenizers, trainers
    from pocketllm_b200.formats import gguf
    corpus = ["The quick brown fox jumps over the lazy dog.", "It's 2024, isn't it? We've seen 1,234 things; they'll see more!",
              "def f(x):\n    return x * 2  # twice\n\n", "naïve café über straße", "hello world hello there general kenobi"] * 3
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=400, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), special_tokens=["<|eos|>"]))
    model = json.loads(tok.to_str())["model"]
    tokens = [k for k, _ in sorted(model["vocab"].items(), key=lambda kv: kv[1])]
    merges = [m if isinstance(m, str) else " ".join(m) for m in model["merges"]]
    w = gguf.GGUFWriter()
    w.add_meta("general.architecture", "minimax-m2")
    w.add_meta("tokenizer.ggml.model", "gpt2")
    w.add_meta("tokenizer.ggml.tokens", tokens)
    w.add_meta("tokenizer.ggml.merges", merges)
    w.add_meta("tokenizer.ggml.token_type", [3 if t == "<|eos|>" else 1 for t in tokens])
    w.add_tensor("dummy", np.zeros(32, np.float32), "f32")
    path = tmp_path / "tok.gguf"
    w.write(path)
    return path


@pytest.mark.skipif(GXX is None, reason="no g++")
@pytest.mark.parametrize("flags", ["-fsanitize=address,undefined -fno-sanitize-recover=all", "-fsanitize=thread"])
def test_host_selftest_under_sanitizers(tmp_path, flags):
    exe = tmp_path / "host_selftest"
    cmd = [GXX, "-std=c++17", "-O1", "-g", "-pthread", *flags.split(), *map(str, SRC), "-o", str(exe)]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if b.returncode != 0 and ("cannot find -l" in b.stderr or "libasan" in b.stderr or "libtsan" in b.stderr or "libubsan" in b.stderr):
        pytest.skip("sanitizer runtime is not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    r = subprocess.run([str(exe), *_inputs(tmp_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "host_selftest=ok" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


@pytest.mark.skipif(GXX is None, reason="no g++")
def test_kv_swap_tier_and_lru_map_host_only_under_asan(tmp_path):
    """The KV swap tier in its host-only mode and the LRU slot map under AddressSanitizer + UBSan. The CUDA runtime is
    linked (the sources also hold the device paths) but never called."""
    cuda = Path("/usr/local/cuda")
    if not (cuda / "include" / "cuda_runtime.h").exists() or not list((cuda / "lib64").glob("libcudart.so*")):
        pytest.skip("CUDA toolkit headers / runtime not found")
    eng = ROOT / "csrc" / "engine"
    exe = tmp_path / "host_swap_selftest"
    cmd = [GXX, "-std=c++17", "-O1", "-g", "-pthread", "-fsanitize=address,undefined", "-fno-sanitize-recover=all", f"-I{cuda / 'include'}",
           str(ROOT / "csrc" / "tests" / "host_swap_selftest.cpp"), str(eng / "kv_swap.cpp"), str(eng / "staging.cpp"), f"-L{cuda / 'lib64'}",
           "-lcudart", f"-Wl,-rpath,{cuda / 'lib64'}", "-o", str(exe)]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if b.returncode != 0 and ("cannot find -l" in b.stderr or "libasan" in b.stderr or "libubsan" in b.stderr):
        pytest.skip("sanitizer or CUDA runtime library is not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env={"ASAN_OPTIONS": "protect_shadow_gap=0:detect_leaks=0"})
    assert r.returncode == 0 and "host_swap_selftest=ok" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


@pytest.mark.skipif(GXX is None, reason="no g++")
@pytest.mark.parametrize("mode", ["scripted", "worker"])
def test_openai_front_end_under_asan(tmp_path, mode):
    """The C++ OpenAI front end built with AddressSanitizer + UBSan and driven over HTTP: plain and streamed completions,
    log-probability reports, a lost step, a bad request; with its scripted engine and with a Python model worker."""
    import http.client
    import json
    import os
    import sys
    eng = ROOT / "csrc" / "engine"
    exe = tmp_path / "host_server_selftest"
    cmd = [GXX, "-std=c++17", "-O1", "-g", "-pthread", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
           str(ROOT / "csrc" / "tests" / "host_server_selftest.cpp"), *(str(eng / f) for f in ("openai_server.cpp", "http_server.cpp", "json.cpp", "sampler.cpp")),
           "-o", str(exe)]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if b.returncode != 0 and ("cannot find -l" in b.stderr or "libasan" in b.stderr or "libubsan" in b.stderr):
        pytest.skip("sanitizer runtime is not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""), ASAN_OPTIONS="detect_leaks=0")
    proc = subprocess.Popen([str(exe), sys.executable, mode, "Hello ☠ world"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    try:
        line = proc.stdout.readline()
        assert line.startswith("openai_server_listening"), (line, proc.stderr.read() if proc.poll() is not None else "")
        port = int(dict(kv.split("=") for kv in line.split()[1:])["port"])

        def post(body, path="/v1/chat/completions"):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
            c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
            r = c.getresponse()
            data = r.read().decode()
            c.close()
            return r.status, data

        chat = {"messages": [{"role": "user", "content": "hi"}]}
        st, data = post(dict(chat, max_tokens=5))
        assert st == 200 and json.loads(data)["choices"][0]["message"]["content"] == "Hello"
        st, data = post(dict(chat, max_tokens=3, logprobs=True, top_logprobs=2))
        assert st == 200 and [e["token"] for e in json.loads(data)["choices"][0]["logprobs"]["content"]] == ["H", "e", "l"]
        st, data = post(dict(chat, max_tokens=4, stream=True, stream_options={"include_usage": True}))
        assert st == 200 and "data: [DONE]" in data and '"content":"H"' in data.replace(" ", "")
        st, data = post(dict(chat, max_tokens=30))                          # runs into the scripted step failure
        assert st == 500 and json.loads(data)["error"]["type"] == "engine_error"
        assert post({"messages": []})[0] == 400 and post(dict(chat, max_tokens=100000))[0] == 400
        assert post(dict(chat, max_tokens=2))[0] == 200                     # and serves on
        # malformed traffic must not bring the process down (or trip the sanitizers)
        import socket
        for raw in (b"GARBAGE\r\n\r\n", b"POST /v1/chat/completions HTTP/1.1\r\nContent-Length: 999999\r\n\r\n{\"messages\"",
                    b"GET /" + b"a" * 70000 + b" HTTP/1.1\r\n\r\n", b"POST /v1/chat/completions HTTP/1.1\r\nContent-Length: -5\r\n\r\n",
                    b"POST /v1/chat/completions HTTP/1.1\r\nContent-Length: 7\r\n\r\nnotjson", b"\x00\xff\xfe" * 100, b""):
            with socket.create_connection(("127.0.0.1", port), timeout=10) as so:
                so.settimeout(3)
                if raw:
                    so.sendall(raw)
                try:
                    so.shutdown(socket.SHUT_WR)
                    while so.recv(65536):
                        pass
                except OSError:
                    pass
        assert post(dict(chat, max_tokens=2))[0] == 200
        post({}, "/shutdown")
        proc.wait(timeout=60)
        out, err = proc.stdout.read(), proc.stderr.read()
        assert proc.returncode == 0 and "host_server_selftest=ok" in out, (out[-2000:], err[-4000:])
    finally:
        if proc.poll() is None:
            proc.kill()
            proc.wait(timeout=20)
