"""The native CLI's OpenAI server (HTTP + SSE + Python sidecar) with its scripted engine, the native GGUF
reader and the host sampler: everything here runs without a GPU."""
import ctypes
import http.client
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
BINARY = ROOT / "pocketllm_b200" / "_C" / "pocket_engine"

pytestmark = pytest.mark.skipif(not BINARY.exists(), reason="pocket_engine is not built")


class Server:
    def __init__(self, script: str, max_context: int = 4096):
        env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
        self.proc = subprocess.Popen(
            [str(BINARY), "--serve", "--port", "0", "--fake-engine-script", script, "--tokenizer", "chars", "--chat-format", "dsv4",
             "--sidecar-python", sys.executable, "--allow-shutdown", "--max-context", str(max_context), "--model-name", "scripted"],
            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
        line = self.proc.stdout.readline()
        assert line.startswith("openai_server_listening"), (line, self.proc.stderr.read() if self.proc.poll() is not None else "")
        self.port = int(dict(kv.split("=") for kv in line.split()[1:])["port"])

    def request(self, method, path, body=None):
        c = http.client.HTTPConnection("127.0.0.1", self.port, timeout=60)
        c.request(method, path, None if body is None else json.dumps(body), {"Content-Type": "application/json"})
        r = c.getresponse()
        data = r.read().decode()
        c.close()
        return r.status, r.getheader("Content-Type"), data

    def close(self):
        try:
            self.request("POST", "/shutdown", {})
            self.proc.wait(timeout=20)
        except Exception:
            self.proc.kill()
            self.proc.wait(timeout=20)


@pytest.fixture
def server(request):
    s = Server(getattr(request, "param", "Hello, world!"))
    yield s
    s.close()


def _chat(content="hi", **kw):
    return dict({"model": "scripted", "messages": [{"role": "user", "content": content}]}, **kw)


def test_health_models_and_errors(server):
    assert server.request("GET", "/health")[0] == 200
    st, ct, data = server.request("GET", "/v1/models")
    assert st == 200 and "json" in ct and json.loads(data)["data"][0]["id"] == "scripted"
    assert server.request("GET", "/nope")[0] == 404
    assert server.request("GET", "/v1/chat/completions")[0] == 405
    st, _, data = server.request("POST", "/v1/chat/completions", {"messages": []})
    assert st == 400 and "messages" in json.loads(data)["error"]["message"]
    st, _, data = server.request("POST", "/v1/chat/completions", _chat(max_tokens=100000))
    assert st == 400 and json.loads(data)["error"]["type"] == "context_length_exceeded"


def test_completion_stop_string_and_length(server):
    st, _, data = server.request("POST", "/v1/chat/completions", _chat())
    out = json.loads(data)
    assert st == 200 and out["object"] == "chat.completion"
    assert out["choices"][0]["message"] == {"role": "assistant", "content": "Hello, world!"}
    assert out["choices"][0]["finish_reason"] == "stop"
    u = out["usage"]
    assert u["completion_tokens"] == len("Hello, world!") + 1 and u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]
    out = json.loads(server.request("POST", "/v1/chat/completions", _chat(stop=["wor"]))[2])
    assert out["choices"][0]["message"]["content"] == "Hello, " and out["choices"][0]["finish_reason"] == "stop"
    out = json.loads(server.request("POST", "/v1/chat/completions", _chat(max_tokens=3))[2])
    assert out["choices"][0]["message"]["content"] == "Hel" and out["choices"][0]["finish_reason"] == "length"


def test_streaming_chunks(server):
    st, ct, data = server.request("POST", "/v1/chat/completions", _chat(stream=True, stream_options={"include_usage": True}))
    assert st == 200 and ct.startswith("text/event-stream")
    events = [e[len("data: "):] for e in data.split("\n\n") if e.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"}
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks if c["choices"])
    assert text == "Hello, world!"
    assert [c["choices"][0]["finish_reason"] for c in chunks if c["choices"]][-1] == "stop"
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == len(text) + 1
    assert all(c["id"] == chunks[0]["id"] and c["object"] == "chat.completion.chunk" for c in chunks)


TOOL_SCRIPT = ('Let me check.\n\n<｜DSML｜tool_calls>\n<｜DSML｜invoke name="get_weather">\n'
               '<｜DSML｜parameter name="city" string="true">Paris</｜DSML｜parameter>\n'
               '<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>\n</｜DSML｜invoke>\n</｜DSML｜tool_calls>')


@pytest.mark.parametrize("server", [TOOL_SCRIPT], indirect=True)
def test_tool_calls_are_parsed_by_the_sidecar(server):
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]
    out = json.loads(server.request("POST", "/v1/chat/completions", _chat("weather?", tools=tools))[2])
    ch = out["choices"][0]
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["content"] == "Let me check."
    call = ch["message"]["tool_calls"][0]["function"]
    assert call["name"] == "get_weather" and json.loads(call["arguments"]) == {"city": "Paris", "days": 3}


@pytest.mark.parametrize("server", ["because</think>42"], indirect=True)
def test_reasoning_goes_to_its_own_channel(server):
    out = json.loads(server.request("POST", "/v1/chat/completions", _chat("why?", reasoning_effort="high"))[2])
    msg = out["choices"][0]["message"]
    assert msg["content"] == "42" and msg["reasoning_content"] == "because"
    data = server.request("POST", "/v1/chat/completions", _chat("why?", reasoning_effort="high", stream=True))[2]
    chunks = [json.loads(e[6:]) for e in data.split("\n\n") if e.startswith("data: {")]
    assert "".join(c["choices"][0]["delta"].get("reasoning_content", "") for c in chunks if c["choices"]) == "because"


@pytest.mark.parametrize("server", ["ab\u2620cd"], indirect=True)
def test_step_failure_ends_the_request_with_500_and_the_next_request_is_served(server):
    """An engine step whose result is lost (a rank's peer wait ran out) must not produce tokens: plain requests get
    HTTP 500, streams an error event, and the server keeps serving."""
    st, _, data = server.request("POST", "/v1/chat/completions", _chat())
    assert st == 500 and json.loads(data)["error"]["type"] == "engine_error"
    st, ct, data = server.request("POST", "/v1/chat/completions", _chat(stream=True))
    assert st == 200 and "event-stream" in ct
    events = [e[6:] for e in data.split("\n\n") if e.startswith("data: ")]
    assert events[-1] == "[DONE]" and any('"engine_error"' in e for e in events)
    text = "".join(json.loads(e)["choices"][0]["delta"].get("content", "") for e in events if e.startswith("{") and "choices" in e)
    assert text in ("", "a", "ab")           # nothing after the failed step
    assert server.request("GET", "/health")[0] == 200


def test_native_gguf_inspect(tmp_path):
    from pocketllm_b200.models import minimax_m2
    p = tmp_path / "mm.gguf"
    minimax_m2.write_random_gguf(p, minimax_m2.MiniMaxM2Config.tiny())
    out = subprocess.run([str(BINARY), "--inspect-gguf", str(p), "--tensors"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    head = dict(kv.split("=") for kv in out.stdout.splitlines()[0].split())
    from pocketllm_b200.formats import gguf
    ref = gguf.GGUFFile(p)
    assert head["architecture"] == "minimax-m2" and int(head["tensors"]) == len(ref.tensors) and int(head["file_bytes"]) == p.stat().st_size
    types = {l.split()[0].split("=")[1]: int(l.split()[2].split("=")[1]) for l in out.stdout.splitlines() if l.startswith("type=")}
    want = {}
    for t in ref.tensors.values():
        want[t.type_name] = want.get(t.type_name, 0) + t.nbytes
    assert types == want
    line = next(l for l in out.stdout.splitlines() if l.startswith("token_embd.weight "))
    t = ref.tensors["token_embd.weight"]
    assert f"bytes={t.nbytes}" in line
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(p.read_bytes()[:200])
    assert subprocess.run([str(BINARY), "--inspect-gguf", str(bad)], capture_output=True, text=True).returncode == 1


def test_native_gguf_reader_rejects_hostile_sizes(tmp_path):
    """Lengths, counts, dimensions and offsets near 2^64 must be refused with a message, not wrapped into range."""
    import struct

    def header(n_tensors: int, n_kv: int) -> bytes:
        return struct.pack("<IIQQ", 0x46554747, 3, n_tensors, n_kv)

    def kv_str(key: str, length: int, payload: bytes = b"") -> bytes:
        return struct.pack("<Q", len(key)) + key.encode() + struct.pack("<IQ", 8, length) + payload

    def tensor(name: str, dims: list[int], typ: int, offset: int) -> bytes:
        return (struct.pack("<Q", len(name)) + name.encode() + struct.pack("<I", len(dims)) +
                b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, offset))

    cases = {
        "string length wraps": header(0, 1) + kv_str("k", 2**64 - 8),
        "array count huge": header(0, 1) + struct.pack("<Q", 1) + b"a" + struct.pack("<IIQ", 9, 4, 2**62),
        "tensor count huge": header(2**60, 0),
        "dims overflow": header(1, 0) + tensor("t", [2**33, 2**33], 0, 0) + b"\0" * 64,
        "offset wraps": header(1, 0) + tensor("t", [32], 0, 2**64 - 32) + b"\0" * 256,
        "past the end": header(1, 0) + tensor("t", [1024], 0, 0) + b"\0" * 64,
    }
    for what, blob in cases.items():
        f = tmp_path / "h.gguf"
        f.write_bytes(blob)
        r = subprocess.run([str(BINARY), "--inspect-gguf", str(f)], capture_output=True, text=True, timeout=60)
        assert r.returncode == 1 and "gguf:" in (r.stdout + r.stderr), (what, r.stdout, r.stderr)


def _engine_lib():
    from pocketllm_b200.ops import lib
    return lib.engine()


def test_host_sampler_greedy_temperature_top_p():
    L = _engine_lib()
    logits = np.array([0.1, 2.0, 2.0, -1.0, 1.5, 0.0], dtype=np.float32)
    ptr = logits.ctypes.data_as(ctypes.c_void_p)
    rng = ctypes.c_uint64(12345)
    call = lambda t, p, k: L.pk_sample_token(ptr, ctypes.c_int(len(logits)), ctypes.c_float(t), ctypes.c_float(p), ctypes.c_int(k), ctypes.byref(rng))
    assert call(0.0, 1.0, 0) == 1                                   # greedy, lowest index on ties
    draws = np.bincount([call(1.0, 1.0, 0) for _ in range(20000)], minlength=6) / 20000
    want = np.exp(logits) / np.exp(logits).sum()
    assert np.abs(draws - want).max() < 0.02
    draws = np.bincount([call(1.0, 0.6, 0) for _ in range(5000)], minlength=6)
    assert draws[[0, 3, 5]].sum() == 0 and draws[1] > 0 and draws[2] > 0          # nucleus keeps the head only
    draws = np.bincount([call(0.7, 1.0, 2) for _ in range(2000)], minlength=6)
    assert draws[[0, 3, 4, 5]].sum() == 0


def test_native_gguf_reader_matches_python_reader(tmp_path):
    from pocketllm_b200.formats import gguf
    from pocketllm_b200.models import glm_dsa
    p = tmp_path / "glm.gguf"
    glm_dsa.write_random_gguf(p, glm_dsa.GLMDSAConfig.tiny())
    L = _engine_lib()
    L.pk_gguf_describe.restype = ctypes.c_char_p
    d = json.loads(L.pk_gguf_describe(str(p).encode()))
    ref = gguf.GGUFFile(p)
    assert d["version"] == 3 and d["metadata"]["general.architecture"] == "glm-dsa"
    for k, v in ref.metadata.items():
        got = d["metadata"][k]
        if isinstance(v, float):
            assert abs(got - v) < 1e-6 * max(1.0, abs(v)), k
        elif isinstance(v, (int, str, bool)):
            assert got == v, k
        else:
            assert list(got) == list(v), k
    assert [t["name"] for t in d["tensors"]] == list(ref.tensors)
    for t in d["tensors"]:
        r = ref.tensors[t["name"]]
        assert t["type"] == r.type_name and t["nbytes"] == r.nbytes and tuple(reversed(t["dims"])) == tuple(r.shape)
        assert t["head_sum"] == int(np.frombuffer(ref.raw(t["name"]).tobytes()[:64], dtype=np.uint8).sum())
    assert L.pk_gguf_describe(str(tmp_path / "missing.gguf").encode()) is None


def test_sidecar_plan_carries_every_sampling_field_the_native_sampler_reads():
    from pocketllm_b200.server import cpp_sidecar as sc
    s = sc.Session(sc.CharTokenizer())
    plan = s.begin({"messages": [{"role": "user", "content": "hi"}], "temperature": 0.7, "top_p": 0.9, "top_k": 40, "min_p": 0.05,
                    "frequency_penalty": 0.3, "presence_penalty": 0.2, "repetition_penalty": 1.1, "seed": 7, "max_tokens": 9})
    assert plan["ok"] and plan["max_tokens"] == 9 and plan["seed"] == 7
    for key, want in (("temperature", 0.7), ("top_p", 0.9), ("top_k", 40), ("min_p", 0.05), ("frequency_penalty", 0.3),
                      ("presence_penalty", 0.2), ("repetition_penalty", 1.1)):
        assert plan[key] == pytest.approx(want), key
    bad = s.begin({"messages": [{"role": "user", "content": "hi"}], "n": 2})
    assert not bad["ok"] and bad["status"] == 400


def test_logprobs_of_every_generated_token(server):
    st, _, data = server.request("POST", "/v1/chat/completions", _chat(max_tokens=3, logprobs=True, top_logprobs=2))
    out = json.loads(data)
    assert st == 200, data
    content = out["choices"][0]["logprobs"]["content"]
    assert [e["token"] for e in content] == ["H", "e", "l"] and out["choices"][0]["message"]["content"] == "Hel"
    for e in content:
        assert e["logprob"] == pytest.approx(-0.6931472, rel=1e-5) and e["bytes"] == [ord(e["token"])]
        assert [t["token"] for t in e["top_logprobs"]] == [e["token"], chr(ord(e["token"]) + 1)]
        assert e["top_logprobs"][1]["logprob"] == pytest.approx(-1.3862944, rel=1e-5)
    # logprobs without alternatives, none when not asked for, and the refusals of the request validation
    out = json.loads(server.request("POST", "/v1/chat/completions", _chat(max_tokens=2, logprobs=True))[2])
    assert [e["top_logprobs"] for e in out["choices"][0]["logprobs"]["content"]] == [[], []]
    assert "logprobs" not in json.loads(server.request("POST", "/v1/chat/completions", _chat(max_tokens=2))[2])["choices"][0]
    assert server.request("POST", "/v1/chat/completions", _chat(logprobs=True, stream=True))[0] == 400
    assert server.request("POST", "/v1/chat/completions", _chat(top_logprobs=3))[0] == 400


class WorkerServer(Server):
    """The native front end in front of a Python model worker (here the worker's scripted stand-in model)."""

    def __init__(self, script: str):
        env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
        self.proc = subprocess.Popen(
            [str(BINARY), "--serve", "--port", "0", "--model-worker", "scripted", "--worker-script", script, "--tokenizer", "chars", "--chat-format", "dsv4",
             "--sidecar-python", sys.executable, "--allow-shutdown", "--max-context", "512", "--model-name", "worker"],
            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
        line = self.proc.stdout.readline()
        assert line.startswith("openai_server_listening") and "engine=worker" in line, (line, self.proc.stderr.read() if self.proc.poll() is not None else "")
        self.port = int(dict(kv.split("=") for kv in line.split()[1:])["port"])


def test_native_front_end_serves_a_python_model_worker():
    s = WorkerServer("Bonjour ☠ monde")
    try:
        out = json.loads(s.request("POST", "/v1/chat/completions", _chat(max_tokens=7))[2])
        assert out["choices"][0]["message"]["content"] == "Bonjour" and out["choices"][0]["finish_reason"] == "length"
        out = json.loads(s.request("POST", "/v1/chat/completions", _chat(max_tokens=3, logprobs=True, top_logprobs=1))[2])
        content = out["choices"][0]["logprobs"]["content"]
        assert [e["token"] for e in content] == ["B", "o", "n"] and content[0]["logprob"] == pytest.approx(-0.6931472, rel=1e-5)
        assert [t["token"] for t in content[1]["top_logprobs"]] == ["o"]
        # the worker's step failure (a lost step) ends the request with 500; the next request is served
        st, _, data = s.request("POST", "/v1/chat/completions", _chat(max_tokens=20))
        assert st == 500 and json.loads(data)["error"]["type"] == "engine_error"
        assert s.request("POST", "/v1/chat/completions", _chat(max_tokens=2))[0] == 200
        # the context limit comes from the worker
        assert s.request("POST", "/v1/chat/completions", _chat(max_tokens=100000))[0] == 400
    finally:
        s.close()


def test_model_worker_protocol_in_process():
    import io
    from pocketllm_b200.server import model_worker as mw
    reqs = [{"op": "hello"}, {"op": "next"}, {"op": "prefill", "tokens": [1, 2], "sampler": {"logprobs": 1}}, {"op": "next"}, {"op": "next"},
            {"op": "next"}, {"op": "bogus"}, {"op": "quit"}, {"op": "hello"}]
    out = io.StringIO()
    mw.serve(mw.ScriptedBackend("ab"), "scripted", 64, stdin=io.StringIO("".join(json.dumps(r) + "\n" for r in reqs)), stdout=out)
    replies = [json.loads(l) for l in out.getvalue().splitlines()]
    assert len(replies) == 7                                              # nothing after quit
    assert replies[0] == {"ok": True, "max_context": 64, "model": "scripted"}
    assert "next before prefill" in replies[1]["error"] and replies[1]["lost"] is False
    assert replies[2]["token"] == ord("a") and replies[2]["top"] == [[ord("a"), pytest.approx(-0.6931472)]]
    assert replies[3]["token"] == ord("b") and replies[4]["token"] == 0 and replies[5] == {"token": 0, "done": True}
    assert "unknown op" in replies[6]["error"]


def test_model_worker_on_two_ranks_follows_rank_zero(tmp_path):
    """The worker under torchrun (gloo, CPU): rank 0 answers on the pipe, rank 1 follows every request to the step where
    the limits end it."""
    import socket
    with socket.socket() as so:
        so.bind(("127.0.0.1", 0))
        port = so.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    reqs = [{"op": "hello"}, {"op": "prefill", "tokens": [1, 2, 3], "sampler": {}, "max_tokens": 3, "stop_token_ids": [0]}, {"op": "next"},
            {"op": "prefill", "tokens": [4], "sampler": {}, "max_tokens": 50, "stop_token_ids": [ord("l")]}, {"op": "next"}, {"op": "next"}, {"op": "quit"}]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), "-m", "pocketllm_b200.server.model_worker", "--model", "scripted", "--script", "Hello", "--max-context", "64"],
                       input="".join(json.dumps(q) + "\n" for q in reqs), capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stderr[-3000:]
    replies = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert replies[0]["ok"] and [x["token"] for x in replies[1:3]] == [ord("H"), ord("e")]
    assert [x["token"] for x in replies[3:6]] == [ord("H"), ord("e"), ord("l")]
    assert "rank 1: followed 2 requests" in r.stderr
