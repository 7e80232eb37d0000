"""OpenAI server behaviours over real HTTP with a fake engine and tokenizer (CPU): JSON and SSE
responses, stop strings, thinking content, tool calls, validation errors, context limit."""
import json
import threading
import urllib.error
import urllib.request

import pytest

from pocketllm_b200.encoding import dsv4
from pocketllm_b200.server import openai as oa
from pocketllm_b200.server.engine import SamplingParams, ServingEngine, sample_token


class CharTokenizer:
    """One token per character (ids = code points); id 0 is EOS."""
    eos_ids = (0,)

    def __init__(self):
        self.last_prompt = None

    def encode_chat(self, messages, *, tools=None, thinking=False, reasoning_effort=None, response_format=None):
        self.last_prompt = dsv4.encode_messages(messages, tools=tools, thinking_mode="thinking" if thinking else "chat",
                                                reasoning_effort=reasoning_effort, response_format=response_format)
        return [ord(c) for c in self.last_prompt]

    def decode(self, ids):
        return "".join(chr(i) for i in ids)

    def parse(self, text, thinking):
        return dsv4.parse_completion(("" if thinking else "</think>") + text if not thinking else "<think>" + text, "thinking" if thinking else "chat")


class ScriptedBackend:
    def __init__(self, script: str):
        self.script = script
        self.calls = []

    def generate(self, prompt_ids, params: SamplingParams):
        self.calls.append((len(prompt_ids), params))
        for ch in self.script:
            yield ord(ch)
        yield 0


@pytest.fixture
def server():
    made = []

    def make(script, max_context=4096):
        backend = ScriptedBackend(script)
        app = oa.OpenAIApp(ServingEngine(backend), CharTokenizer(), model_name="fake", max_context=max_context)
        httpd = oa.serve(app, "127.0.0.1", 0)
        threading.Thread(target=httpd.serve_forever, daemon=True).start()
        made.append((httpd, app))
        return f"http://127.0.0.1:{httpd.server_address[1]}", backend, app
    yield make
    for httpd, app in made:
        httpd.shutdown()
        app.engine.close()


def _post(url, body):
    req = urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=20) as r:
            return r.status, r.read().decode()
    except urllib.error.HTTPError as e:
        return e.code, e.read().decode()


def test_health_models_and_completion(server):
    url, backend, app = server("Hello there")
    assert json.loads(urllib.request.urlopen(url + "/health").read())["status"] == "ok"
    assert json.loads(urllib.request.urlopen(url + "/v1/models").read())["data"][0]["id"] == "fake"
    code, text = _post(url, {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 64})
    d = json.loads(text)
    assert code == 200 and d["choices"][0]["message"]["content"] == "Hello there"
    assert d["choices"][0]["finish_reason"] == "stop"
    assert d["usage"]["completion_tokens"] == len("Hello there") + 1 and d["usage"]["prompt_tokens"] == backend.calls[0][0]
    assert d["timings"]["prefill_seconds"] is not None


def test_stop_string_and_max_tokens(server):
    url, _, _ = server("abcSTOPdef")
    _, text = _post(url, {"messages": [{"role": "user", "content": "x"}], "stop": ["STOP"]})
    d = json.loads(text)
    assert d["choices"][0]["message"]["content"] == "abc" and d["choices"][0]["finish_reason"] == "stop"
    _, text = _post(url, {"messages": [{"role": "user", "content": "x"}], "max_tokens": 4})
    d = json.loads(text)
    assert d["choices"][0]["message"]["content"] == "abcS" and d["choices"][0]["finish_reason"] == "length"


def test_streaming_sse_with_thinking_and_tools(server):
    call = [{"type": "function", "function": {"name": "f", "arguments": json.dumps({"a": 1})}}]
    script = "think hard</think>Answer.\n\n" + dsv4.render_tool_calls(call)
    url, _, _ = server(script)
    code, text = _post(url, {"messages": [{"role": "user", "content": "x"}], "stream": True, "reasoning_effort": "high",
                             "stream_options": {"include_usage": True},
                             "tools": [{"type": "function", "function": {"name": "f", "parameters": {}}}]})
    assert code == 200
    events = [json.loads(l[6:]) for l in text.split("\n\n") if l.startswith("data: {")]
    assert text.strip().endswith("data: [DONE]")
    reasoning = "".join(e["choices"][0]["delta"].get("reasoning_content", "") for e in events)
    content = "".join(e["choices"][0]["delta"].get("content", "") for e in events)
    assert reasoning == "think hard" and content.startswith("Answer.")
    tool_events = [e for e in events if "tool_calls" in e["choices"][0]["delta"]]
    assert tool_events and tool_events[0]["choices"][0]["delta"]["tool_calls"][0]["function"]["name"] == "f"
    assert events[-1]["choices"][0]["finish_reason"] == "tool_calls" and events[-1]["usage"]["completion_tokens"] > 0


def test_validation_errors_and_context_limit(server):
    url, _, _ = server("x", max_context=64)
    for body in ({"messages": []}, {"messages": [{"role": "user", "content": "x"}], "stream": True, "n": 2},
                 {"messages": [{"role": "user", "content": "x"}], "max_tokens": 0},
                 {"messages": [{"role": "user", "content": "x"}], "stream": True, "logprobs": True},
                 {"messages": [{"role": "user", "content": "y" * 200}]}):
        code, text = _post(url, body)
        assert code == 400 and "error" in json.loads(text)
    req = urllib.request.Request(url + "/v1/chat/completions", data=b"{not json", headers={"Content-Type": "application/json"})
    with pytest.raises(urllib.error.HTTPError) as ei:
        urllib.request.urlopen(req)
    assert ei.value.code == 400


def test_streaming_decoder_holds_back_partial_stop():
    tok = CharTokenizer()
    dec = oa.StreamingDecoder(tok, ["END"])
    out = [dec.push(ord(c)) for c in "abEN"]
    assert "".join(out) == "ab"          # "EN" could still become "END"
    assert dec.push(ord("x")) == "ENx"
    out = "".join(dec.push(ord(c)) for c in "yENDz")
    assert out == "y" and dec.stopped and dec.text == "abENxy"


def test_sampler_greedy_and_topk():
    import torch
    logits = torch.tensor([0.1, 3.0, 3.0, -1.0])
    assert sample_token(logits, SamplingParams(temperature=0.0)) == 1
    g = torch.Generator().manual_seed(0)
    picks = {sample_token(logits, SamplingParams(temperature=1.0, top_k=2), g) for _ in range(50)}
    assert picks <= {1, 2}
    picks = {sample_token(logits, SamplingParams(temperature=1.0, top_p=0.3), g) for _ in range(20)}
    assert len(picks) == 1


class LogitBackend:
    """Five-token vocabulary whose logits depend on the step; yields `TokenInfo` when log-probabilities are asked for."""

    def generate(self, prompt_ids, params: SamplingParams):
        import torch
        from pocketllm_b200.server.engine import token_logprobs
        for step in range(params.max_tokens):
            logits = torch.tensor([-9.0, 1.0, 2.0 + step, 0.5, -1.0])
            tok = int(logits.argmax())
            yield token_logprobs(logits, tok, params.logprobs) if params.logprobs >= 0 else tok


class SmallTokenizer(CharTokenizer):
    def decode(self, ids):
        return "".join("?abcd"[i] for i in ids)


def test_logprobs_of_every_generated_token_with_alternatives():
    import math
    import torch
    app = oa.OpenAIApp(ServingEngine(LogitBackend()), SmallTokenizer(), model_name="fake")
    try:
        out = app.complete({"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "logprobs": True, "top_logprobs": 2})
        content = out["choices"][0]["logprobs"]["content"]
        assert [e["token"] for e in content] == ["b", "b", "b"] and out["usage"]["completion_tokens"] == 3
        for step, e in enumerate(content):
            lp = torch.log_softmax(torch.tensor([-9.0, 1.0, 2.0 + step, 0.5, -1.0]), -1)
            assert math.isclose(e["logprob"], float(lp[2]), rel_tol=1e-5) and e["bytes"] == [ord("b")]
            assert [t["token"] for t in e["top_logprobs"]] == ["b", "a"]
            assert math.isclose(e["top_logprobs"][1]["logprob"], float(lp[1]), rel_tol=1e-5)
        # without the flag nothing is added; the flags are validated
        plain = app.complete({"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2})
        assert "logprobs" not in plain["choices"][0]
        for bad in ({"top_logprobs": 3}, {"logprobs": True, "top_logprobs": 21}, {"logprobs": True, "stream": True}):
            with pytest.raises(oa.BadRequest):
                app.complete({"messages": [{"role": "user", "content": "hi"}], **bad}) if not bad.get("stream") else next(app.stream({"messages": [{"role": "user", "content": "hi"}], **bad}))
    finally:
        app.engine.close()


def test_backends_report_logprobs_from_their_logits():
    """The GGUF and DeepSeek-V4 backends over stand-in runtimes that return CPU logits."""
    import torch
    from pocketllm_b200.server.backends import DSV4Backend, GGUFBackend

    class Runtime:
        def __init__(self):
            self.fed = []
            self.combine = type("C", (), {"check_step": staticmethod(lambda dev: None)})()

        def reset(self):
            self.fed = []

        def forward_logits(self, tokens):
            self.fed += list(tokens)
            z = torch.zeros(6)
            z[(len(self.fed) * 2) % 6] = 3.0
            return z

    p = SamplingParams(max_tokens=3, logprobs=1, stop_token_ids=(5,))
    got = list(GGUFBackend(Runtime()).generate([1, 2], p))
    assert [t.token for t in got] == [4, 0, 2] and all(abs(t.logprob - float(torch.log_softmax(torch.tensor([3.0, 0, 0, 0, 0, 0]), -1)[0])) < 1e-6 for t in got)
    assert all(t.top[0][0] == t.token for t in got)

    # a penalised request without log-probabilities also goes through the logits (plain ints come out)
    pen = list(GGUFBackend(Runtime()).generate([1, 2], SamplingParams(max_tokens=3, repetition_penalty=100.0, stop_token_ids=(5,))))
    assert pen[0] == 4 and all(isinstance(t, int) for t in pen) and len(pen) == 3

    class Runtime2(Runtime):
        def forward_logits(self, tokens):
            return super().forward_logits(tokens).unsqueeze(0)          # [rows, vocab]

    got2 = list(DSV4Backend(Runtime2()).generate([1, 2], p))
    assert [t.token for t in got2] == [4, 0, 2]
    plain = list(DSV4Backend(Runtime2()).generate([1, 2], SamplingParams(max_tokens=3)))
    assert plain == [4, 0, 2]
    with pytest.raises(RuntimeError):
        list(GGUFBackend(type("R", (), {"reset": lambda self: None})()).generate([1], p))


def test_server_command_line_takes_profiles_config_files_and_the_reference_flag_names(tmp_path):
    import json
    ck = tmp_path / "ck"
    ck.mkdir()
    (ck / "config.json").write_text(json.dumps({"linear_num_value_heads": 4, "hidden_size": 64}))
    args, st = oa.parse_server_args(["--ckpt-path", str(ck), "--max-model-len", "2048", "--model", "my-model-id"], env={})
    assert st["kind"] == "qwen" and st["model_name"] == "my-model-id" and st["max_context"] == 2048 and st["max_queue"] == 64
    assert st["host"] == "127.0.0.1" and st["port"] == 8000 and not st["layer_pipeline"]
    # a profile from the environment, a config file on top of it, flags on top of that
    cfgf = tmp_path / "serve.json"
    cfgf.write_text(json.dumps({"serving": {"port": 9001, "model_name": "from-file"}, "model": {"max_context": 1024}}))
    args, st = oa.parse_server_args(["--ckpt", str(ck), "--model", "qwen", "--config", str(cfgf), "--port", "9002"],
                                    env={"SERVING_PROFILE": "safe1"})
    assert st["max_queue"] == 1 and st["port"] == 9002 and st["model_name"] == "from-file" and st["max_context"] == 1024 and st["profile"] == "safe1"
    assert st["speculative"] == ("off", 4)
    assert oa.parse_server_args(["--ckpt", str(ck), "--serving-profile", "latency2"], env={})[1]["speculative"] == ("ngram", 4)
    # a directory without DeltaNet fields is a DeepSeek-V4 checkpoint; its layer pipeline is a partition policy
    d4dir = tmp_path / "d4"
    d4dir.mkdir()
    (d4dir / "config.json").write_text(json.dumps({"n_layers": 4}))
    args, st = oa.parse_server_args(["--ckpt", str(d4dir), "--partition-policy", "layer_pp_4gpu"], env={})
    assert st["kind"] == "dsv4" and st["layer_pipeline"]
    with pytest.raises(SystemExit):
        oa.parse_server_args(["--ckpt", str(ck), "--routed-experts-device", "cpu"], env={})
    with pytest.raises(SystemExit):
        oa.parse_server_args([], env={})
    with pytest.raises(ValueError):
        oa.parse_server_args(["--ckpt", str(ck), "--serving-profile", "nope"], env={})


def test_metrics_endpoint_reports_the_engine_counters(server):
    url, backend, app = server("ok")
    assert _post(url, {"messages": [{"role": "user", "content": "x"}]})[0] == 200
    with urllib.request.urlopen(url + "/metrics", timeout=20) as r:
        text = r.read().decode()
        assert r.headers["Content-Type"].startswith("text/plain")
    vals = dict(line.split() for line in text.splitlines() if not line.startswith("#"))
    assert vals["pocketllm_requests_total"] == "1" and int(vals["pocketllm_tokens_total"]) >= 2
    assert vals["pocketllm_errors_total"] == "0" and vals["pocketllm_queue_depth"] == "0"


def test_backend_is_detected_from_a_gguf_files_architecture(tmp_path):
    import numpy as np
    from pocketllm_b200.formats import gguf
    for arch, want in (("deepseek4", "dsv4"), ("minimax-m2", "gguf"), ("glm-dsa", "gguf")):
        w = gguf.GGUFWriter()
        w.add_meta("general.architecture", arch)
        w.add_tensor("token_embd.weight", np.zeros((2, 4), dtype=np.float32), "f32", (2, 4))
        path = tmp_path / f"{arch}.gguf"
        w.write(path)
        assert oa.detect_model_kind(str(path)) == want
        args, st = oa.parse_server_args(["--ckpt", str(path)], env={})
        assert st["kind"] == want


def test_tool_choice_and_parallel_tool_calls_become_instructions():
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {}}}]
    msgs = [{"role": "user", "content": "hi"}]
    assert oa.with_tool_directive(msgs, tools, "auto", None) is msgs and oa.with_tool_directive(msgs, None, "required", False) is msgs
    out = oa.with_tool_directive(msgs, tools, "required", False)
    assert out[0]["role"] == "system" and "must answer by calling one of" in out[0]["content"] and "at most one tool" in out[0]["content"] and out[1:] == msgs
    named = oa.with_tool_directive([{"role": "system", "content": "Be brief."}] + msgs, tools, {"type": "function", "function": {"name": "get_weather"}}, None)
    assert named[0]["content"].startswith("Be brief.") and "`get_weather`" in named[0]["content"] and len(named) == 2
    with pytest.raises(oa.BadRequest):
        oa.with_tool_directive(msgs, tools, {"type": "function", "function": {"name": "nope"}}, None)


def test_qwen_backend_logprob_and_speculator_paths_with_a_stand_in_engine():
    """The Qwen backend's control flow over a stand-in engine: log-probability requests read every step's logits and bypass
    the speculator; plain greedy requests go through the speculator when there is one."""
    import torch
    from pocketllm_b200.server.backends import QwenBackend

    class Engine:
        tp_world = 1

        def __init__(self):
            self.fed, self.calls = [], []

        def reset(self):
            self.fed = []

        def _z(self):
            z = torch.zeros(8)
            z[(sum(self.fed) + len(self.fed)) % 8] = 4.0
            return z

        def prefill(self, tokens):
            self.calls.append("prefill")
            self.fed = list(tokens)
            return int(self._z().argmax())

        def logits(self, row=0):
            return self._z()

        def forward_rows(self, tokens):
            self.calls.append("rows")
            out = []
            for t in tokens:
                self.fed.append(t)
                out.append(int(self._z().argmax()))
            return out

        def decode(self, n, sync_each_step=False):
            self.calls.append("decode")
            out = []
            for _ in range(n):
                out += self.forward_rows([int(self._z().argmax())])
            return out

    class Spec:
        def __init__(self):
            self.used = 0

        def prefill(self, prompt):
            self.used += 1
            return 1

        def decode(self, last, n):
            return [2] * n

    plain = list(QwenBackend(Engine()).generate([1, 2, 3], SamplingParams(max_tokens=4)))
    eng = Engine()
    with_lp = list(QwenBackend(eng).generate([1, 2, 3], SamplingParams(max_tokens=4, logprobs=2)))
    assert [t.token for t in with_lp] == plain and "decode" not in eng.calls
    assert all(t.top[0][0] == t.token and len(t.top) == 2 and t.logprob < 0 for t in with_lp)
    spec = Spec()
    assert list(QwenBackend(Engine(), speculator=spec).generate([1], SamplingParams(max_tokens=3))) == [1, 2, 2] and spec.used == 1
    lp_spec = list(QwenBackend(Engine(), speculator=spec).generate([1, 2, 3], SamplingParams(max_tokens=4, logprobs=0)))
    assert [t.token for t in lp_spec] == plain and spec.used == 1          # log-probabilities: the speculator is bypassed
