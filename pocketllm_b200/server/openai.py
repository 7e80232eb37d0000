"""OpenAI-compatible HTTP server: `GET /health`, `GET /v1/models`,
`POST /v1/chat/completions` (JSON or SSE streaming), with stop strings, thinking /
reasoning content, tool calls, usage and timings.

Surface and behaviours follow the reference's Python server (src/server/openai.py:
payload build 431-640, streaming decoder 643-715, HTTP handler 896-1040) and its C++
twin (cpp_engine/src/openai_server.cpp:179-446): one request in flight, `max_tokens` /
`max_completion_tokens` default 512, `temperature` 0 means greedy, `stream` needs n = 1,
`logprobs` / `top_logprobs` (not with streaming) return the model's log-probability of every generated token and of the most
likely alternatives; the context limit is checked before generation.

    python -m pocketllm_b200.server.openai --model qwen --ckpt DIR [--port 8000]
"""
from __future__ import annotations

import argparse
import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Iterator, Protocol, Sequence

from .engine import SamplingParams, ServingEngine, TokenInfo


class ChatTokenizer(Protocol):
    def encode_chat(self, messages: list[dict], *, tools: list[dict] | None, thinking: bool, reasoning_effort: str | None,
                    response_format: dict | None) -> list[int]: ...
    def decode(self, ids: Sequence[int]) -> str: ...
    def parse(self, text: str, thinking: bool) -> dict: ...
    @property
    def eos_ids(self) -> tuple[int, ...]: ...


class BadRequest(ValueError):
    pass


def build_params(body: dict, eos_ids: tuple[int, ...]) -> tuple[SamplingParams, dict]:
    """Validate an OpenAI chat payload; returns sampling parameters and request options."""
    if not isinstance(body.get("messages"), list) or not body["messages"]:
        raise BadRequest("`messages` must be a non-empty list")
    n = int(body.get("n", 1))
    stream = bool(body.get("stream", False))
    if n < 1 or n > 8:
        raise BadRequest("`n` must be between 1 and 8")
    if stream and n != 1:
        raise BadRequest("`stream` requires n = 1")
    if stream and body.get("logprobs"):
        raise BadRequest("`logprobs` is not available with `stream`")
    top_lp = body.get("top_logprobs")
    if top_lp is not None and (not isinstance(top_lp, int) or not 0 <= top_lp <= 20):
        raise BadRequest("`top_logprobs` must be an integer between 0 and 20")
    if top_lp and not body.get("logprobs"):
        raise BadRequest("`top_logprobs` needs `logprobs` to be true")
    max_tokens = body.get("max_completion_tokens", body.get("max_tokens", 512))
    if not isinstance(max_tokens, int) or max_tokens < 1:
        raise BadRequest("`max_tokens` must be a positive integer")
    stop = body.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    if not all(isinstance(s, str) and s for s in stop) or len(stop) > 16:
        raise BadRequest("`stop` must be a string or up to 16 non-empty strings")
    effort = body.get("reasoning_effort") or (body.get("reasoning") or {}).get("effort")
    thinking = bool(effort) or bool((body.get("reasoning") or {}).get("enabled")) or bool(body.get("thinking"))
    p = SamplingParams(max_tokens=max_tokens, temperature=float(body.get("temperature", 0.0) or 0.0),
                       top_p=float(body.get("top_p", 1.0) or 1.0), top_k=int(body.get("top_k", 0) or 0),
                       min_p=float(body.get("min_p", 0.0) or 0.0), frequency_penalty=float(body.get("frequency_penalty", 0.0) or 0.0),
                       presence_penalty=float(body.get("presence_penalty", 0.0) or 0.0),
                       repetition_penalty=float(body.get("repetition_penalty", 1.0) or 1.0), seed=body.get("seed"),
                       stop_token_ids=tuple(eos_ids), logprobs=int(top_lp or 0) if body.get("logprobs") else -1)
    opts = {"n": n, "logprobs": bool(body.get("logprobs")), "stream": stream, "stop": stop, "thinking": thinking, "reasoning_effort": effort,
            "tools": body.get("tools") if body.get("tool_choice") != "none" else None,
            "response_format": body.get("response_format"),
            "include_usage": bool((body.get("stream_options") or {}).get("include_usage", False))}
    return p, opts


def with_tool_directive(messages: list, tools, tool_choice, parallel_tool_calls) -> list:
    """`tool_choice` = "required" or a named function, and `parallel_tool_calls` = false, are instructions to the model:
    they are folded into the system message (a new one in front when the conversation has none). "auto" and "none" add
    nothing ("none" already removed the tools)."""
    if not tools:
        return messages
    notes = []
    if tool_choice == "required":
        notes.append("You must answer by calling one of the available tools.")
    elif isinstance(tool_choice, dict):
        name = (tool_choice.get("function") or {}).get("name") or tool_choice.get("name")
        if name:
            if name not in {(t.get("function") or t).get("name") for t in tools if isinstance(t, dict)}:
                raise BadRequest(f"`tool_choice` names an unknown tool {name!r}")
            notes.append(f"You must answer by calling the tool `{name}`.")
    if parallel_tool_calls is False:
        notes.append("Call at most one tool in this turn.")
    if not notes:
        return messages
    note = " ".join(notes)
    out = [dict(m) for m in messages]
    for m in out:
        if m.get("role") == "system" and isinstance(m.get("content"), str):
            m["content"] = m["content"] + "\n\n" + note
            return out
    return [{"role": "system", "content": note}] + out


class StreamingDecoder:
    """Incremental detokeniser with stop-string handling: text that could still turn into a
    stop string is held back, and nothing after a stop string is ever emitted."""

    def __init__(self, tokenizer: ChatTokenizer, stop: list[str]):
        self.tok, self.stop = tokenizer, stop
        self.ids: list[int] = []
        self.emitted = 0
        self.text = ""
        self.stopped = False

    def push(self, token: int) -> str:
        if self.stopped:
            return ""
        self.ids.append(token)
        text = self.tok.decode(self.ids)
        if text.endswith("�"):      # incomplete UTF-8 sequence: wait for the next token
            return ""
        self.text = text
        cut = len(text)
        for s in self.stop:
            i = text.find(s, max(0, self.emitted - len(s)))
            if i >= 0:
                cut = min(cut, i)
                self.stopped = True
        if not self.stopped:
            hold = 0
            for s in self.stop:
                for k in range(min(len(s) - 1, len(text)), 0, -1):
                    if text.endswith(s[:k]):
                        hold = max(hold, k)
                        break
            cut = len(text) - hold
        out = text[self.emitted:cut] if cut > self.emitted else ""
        self.emitted = max(self.emitted, cut)
        if self.stopped:
            self.text = text[:cut]
        return out

    def flush(self) -> str:
        if self.stopped:
            return ""
        out = self.text[self.emitted:]
        self.emitted = len(self.text)
        return out


class OpenAIApp:
    """Request logic, independent of the HTTP transport (unit-testable)."""

    def __init__(self, engine: ServingEngine, tokenizer: ChatTokenizer, model_name: str = "pocketllm-b200", max_context: int = 4096):
        self.engine, self.tok, self.model_name, self.max_context = engine, tokenizer, model_name, max_context
        self.inflight = threading.Lock()

    def models(self) -> dict:
        return {"object": "list", "data": [{"id": self.model_name, "object": "model", "owned_by": "pocketllm_b200"}]}

    def _prepare(self, body: dict):
        params, opts = build_params(body, tuple(self.tok.eos_ids))
        messages = with_tool_directive(body["messages"], opts["tools"], body.get("tool_choice"), body.get("parallel_tool_calls"))
        ids = self.tok.encode_chat(messages, tools=opts["tools"], thinking=opts["thinking"],
                                   reasoning_effort=opts["reasoning_effort"], response_format=opts["response_format"])
        if len(ids) + 1 > self.max_context:
            raise BadRequest(f"prompt has {len(ids)} tokens, the context limit is {self.max_context}")
        params.max_tokens = min(params.max_tokens, self.max_context - len(ids))
        return params, opts, ids

    def _run(self, ids: list[int], params: SamplingParams, opts: dict, batchable: bool = False) -> Iterator[tuple[str, Any]]:
        """Yields ("delta", text) pieces and finally ("done", info)."""
        dec = StreamingDecoder(self.tok, opts["stop"])
        t0 = time.perf_counter()
        ttft = None
        n_tok = 0
        finish = "length"
        lps: list[TokenInfo] = []
        for item in self.engine.stream(ids, params, batchable=batchable):
            if isinstance(item, tuple):
                ttft = item[1]
                continue
            n_tok += 1
            if isinstance(item, TokenInfo):
                info_tok, item = item, item.token
                if item not in params.stop_token_ids:
                    lps.append(info_tok)
            if item in params.stop_token_ids:
                finish = "stop"
                break
            piece = dec.push(item)
            if piece:
                yield "delta", piece
            if dec.stopped:
                finish = "stop"
                break
            if n_tok >= params.max_tokens:
                break
        tail = dec.flush()
        if tail:
            yield "delta", tail
        total = time.perf_counter() - t0
        dt = max(total - (ttft or 0.0), 1e-9)
        yield "done", {"finish_reason": finish, "completion_tokens": n_tok, "text": dec.text, "logprobs": lps, "timings": {
            "prefill_seconds": ttft, "decode_seconds": total - (ttft or 0.0), "prompt_tokens_per_second": (len(ids) / ttft) if ttft else None,
            "decode_tokens_per_second": (max(n_tok - 1, 0) / dt) if n_tok > 1 else None}}

    def _logprob_entry(self, t: TokenInfo) -> dict:
        def one(tid: int, lp: float) -> dict:
            text = self.tok.decode([tid])
            return {"token": text, "logprob": lp, "bytes": list(text.encode("utf-8"))}
        entry = one(t.token, t.logprob)
        entry["top_logprobs"] = [one(i, lp) for i, lp in t.top]
        return entry

    def complete(self, body: dict) -> dict:
        params, opts, ids = self._prepare(body)
        choices, completion_tokens, timings = [], 0, None
        # no lock here: whole completions may share a batch in the serving engine, which serialises everything else
        for i in range(opts["n"]):
            info = None
            for kind, val in self._run(ids, params, opts, batchable=not opts["logprobs"]):
                if kind == "done":
                    info = val
            msg = self.tok.parse(info["text"], opts["thinking"])
            finish = "tool_calls" if msg.get("tool_calls") else info["finish_reason"]
            choice = {"index": i, "message": msg, "finish_reason": finish}
            if opts["logprobs"]:
                if not info["logprobs"] and info["completion_tokens"] > 1:
                    raise BadRequest("this model backend does not report log-probabilities")
                choice["logprobs"] = {"content": [self._logprob_entry(t) for t in info["logprobs"]]}
            choices.append(choice)
            completion_tokens += info["completion_tokens"]
            timings = info["timings"]
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()),
                "model": self.model_name, "choices": choices,
                "usage": {"prompt_tokens": len(ids), "completion_tokens": completion_tokens, "total_tokens": len(ids) + completion_tokens},
                "timings": timings, "deepseek_timings": timings}      # the second key is the name the reference's clients read

    def stream(self, body: dict) -> Iterator[str]:
        """SSE lines (`data: {...}\\n\\n`), ending with `data: [DONE]`."""
        params, opts, ids = self._prepare(body)
        cid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())

        def chunk(delta: dict, finish=None, extra=None) -> str:
            d = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": self.model_name,
                 "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
            if extra:
                d.update(extra)
            return "data: " + json.dumps(d, ensure_ascii=False) + "\n\n"

        with self.inflight:
            yield chunk({"role": "assistant", "content": ""})
            in_think = opts["thinking"]
            buf = ""
            info = None
            for kind, val in self._run(ids, params, opts):
                if kind == "done":
                    info = val
                    break
                if in_think:
                    buf += val
                    if "</think>" in buf:
                        r, rest = buf.split("</think>", 1)
                        r = r.replace("<think>", "", 1)
                        if r:
                            yield chunk({"reasoning_content": r})
                        if rest:
                            yield chunk({"content": rest})
                        in_think, buf = False, ""
                    elif len(buf) > 16 and not buf.endswith(("<", "</", "</t", "</th", "</thi", "</thin", "</think")):
                        yield chunk({"reasoning_content": buf.replace("<think>", "", 1)})
                        buf = ""
                else:
                    yield chunk({"content": val})
            if buf:
                yield chunk({"reasoning_content" if in_think else "content": buf})
            msg = self.tok.parse(info["text"], opts["thinking"])
            finish = info["finish_reason"]
            if msg.get("tool_calls"):
                finish = "tool_calls"
                yield chunk({"tool_calls": [dict(tc, index=i) for i, tc in enumerate(msg["tool_calls"])]})
            usage = {"prompt_tokens": len(ids), "completion_tokens": info["completion_tokens"],
                     "total_tokens": len(ids) + info["completion_tokens"]}
            last = {"timings": info["timings"], "deepseek_timings": info["timings"]}
            if opts["include_usage"]:
                last["usage"] = usage
            yield chunk({}, finish, last)
            yield "data: [DONE]\n\n"


def make_handler(app: OpenAIApp):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):  # quiet
            pass

        def _json(self, code: int, obj: dict) -> None:
            data = json.dumps(obj, ensure_ascii=False).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def _error(self, code: int, msg: str, typ: str = "invalid_request_error") -> None:
            self._json(code, {"error": {"message": msg, "type": typ, "code": code}})

        def do_GET(self):
            if self.path == "/health":
                self._json(200, {"status": "ok", "stats": app.engine.stats})
            elif self.path == "/v1/models":
                self._json(200, app.models())
            elif self.path == "/metrics":
                # Prometheus text format: the serving engine's counters
                lines = []
                for key, val in sorted(app.engine.stats.items()):
                    name = f"pocketllm_{key}_total"
                    lines += [f"# TYPE {name} counter", f"{name} {int(val)}"]
                lines += ["# TYPE pocketllm_queue_depth gauge", f"pocketllm_queue_depth {app.engine.queue_depth()}"]
                data = ("\n".join(lines) + "\n").encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)
            else:
                self._error(404, f"no route {self.path}")

        def do_POST(self):
            if self.path != "/v1/chat/completions":
                return self._error(404, f"no route {self.path}")
            try:
                n = int(self.headers.get("Content-Length", "0"))
                body = json.loads(self.rfile.read(n) or b"{}")
            except Exception:
                return self._error(400, "request body is not valid JSON")
            try:
                if body.get("stream"):
                    gen = app.stream(body)
                    first = next(gen)              # validation errors surface before the headers
                    self.send_response(200)
                    self.send_header("Content-Type", "text/event-stream")
                    self.send_header("Cache-Control", "no-cache")
                    self.send_header("Transfer-Encoding", "chunked")
                    self.end_headers()
                    for piece in self._chain(first, gen):
                        data = piece.encode()
                        self.wfile.write(f"{len(data):x}\r\n".encode() + data + b"\r\n")
                        self.wfile.flush()
                    self.wfile.write(b"0\r\n\r\n")
                else:
                    self._json(200, app.complete(body))
            except BadRequest as e:
                self._error(400, str(e))
            except (BrokenPipeError, ConnectionResetError):
                pass
            except Exception as e:
                self._error(500, f"{type(e).__name__}: {e}", "server_error")

        @staticmethod
        def _chain(first, gen):
            yield first
            yield from gen

    return Handler


def serve(app: OpenAIApp, host: str = "127.0.0.1", port: int = 8000) -> ThreadingHTTPServer:
    httpd = ThreadingHTTPServer((host, port), make_handler(app))
    httpd.daemon_threads = True
    return httpd


def detect_model_kind(ckpt: str, ckpt_format: str = "auto") -> str:
    """Backend for a checkpoint path: a GGUF file with the deepseek4 architecture or a DeepSeek-V4 Safetensors directory ->
    `dsv4`, any other GGUF file -> `gguf`, a directory whose config names Gated DeltaNet fields -> `qwen`."""
    from pathlib import Path
    path = Path(ckpt)
    fmt = ckpt_format
    if fmt == "auto":
        fmt = "gguf" if path.suffix == ".gguf" else "safetensors"
    if fmt == "gguf":
        from ..formats import gguf
        arch = gguf.GGUFFile(gguf.shard_paths(str(path))[0]).architecture()
        return "dsv4" if arch == "deepseek4" else "gguf"
    cfg_file = path / "config.json"
    text = cfg_file.read_text() if cfg_file.exists() else "{}"
    return "qwen" if ("linear_num_value_heads" in text or "linear_num_key_heads" in text) else "dsv4"


def parse_server_args(argv=None, env=None):
    """Command line of the Python server -> (args, settings). Besides this package's own flags it takes the names of the
    reference's server (src/server/openai.py:1080-1093: --ckpt-path, --ckpt-format, --tokenizer-path, --config,
    --max-model-len, --partition-policy, --pd-mode, --routed-experts-device) and its profile variable SERVING_PROFILE.
    `settings` come from the typed config: defaults < profile < file < environment < flags."""
    import os
    from ..config import Config
    env = os.environ if env is None else env
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None, help="backend (qwen | gguf | dsv4; default: detected from the checkpoint) or, for any other "
                                                  "value, the model id reported by /v1/models")
    ap.add_argument("--ckpt", "--ckpt-path", dest="ckpt", default=env.get("CKPT_PATH"))
    ap.add_argument("--ckpt-format", choices=["auto", "safetensors", "gguf"], default=env.get("CKPT_FORMAT", "auto"))
    ap.add_argument("--tokenizer-path", default=env.get("TOKENIZER_PATH"), help="directory with tokenizer.json when it is not the checkpoint's")
    ap.add_argument("--config", default=None, help="JSON / YAML file of the typed configuration (sections model, parallel, cache, speculative, serving)")
    ap.add_argument("--serving-profile", default=env.get("SERVING_PROFILE"), help="safe1 | latency2 | throughput4")
    ap.add_argument("--model-name", default=None)
    ap.add_argument("--host", default=None)
    ap.add_argument("--port", type=int, default=None)
    ap.add_argument("--max-context", "--max-model-len", dest="max_context", type=int, default=None)
    ap.add_argument("--partition-policy", default=env.get("PARTITION_POLICY", "legacy"),
                    help="dsv4 under several ranks: legacy / baseline_4gpu = routed experts split over the ranks, layer_pp / layer_pp_4gpu = "
                         "contiguous layer ranges per rank (layer pipeline)")
    ap.add_argument("--pd-mode", choices=["off", "scheduler"], default="off",
                    help="accepted for compatibility: requests run one at a time on the GPUs, so there is no CPU expert server to pause between phases")
    ap.add_argument("--routed-experts-device", choices=["gpu", "cpu"], default="gpu")
    ap.add_argument("--qwen-dspark", default="", help="qwen: directory of an external DSpark block drafter; greedy requests run as speculative rounds")
    args = ap.parse_args(argv)
    if not args.ckpt:
        ap.error("--ckpt (or --ckpt-path / CKPT_PATH) is required")
    if args.routed_experts_device == "cpu":
        ap.error("--routed-experts-device cpu: routed experts run on the GPUs here (experts beyond HBM are staged from pinned host memory)")
    cfg = Config.load(args.config, profile=args.serving_profile or None, env=env)
    kinds = ("qwen", "gguf", "dsv4")
    kind = args.model if args.model in kinds else detect_model_kind(args.ckpt, args.ckpt_format)
    name = args.model_name or (args.model if args.model and args.model not in kinds else None) or cfg.serving.model_name
    settings = {"kind": kind, "model_name": name, "host": args.host or cfg.serving.host, "port": args.port if args.port is not None else cfg.serving.port,
                "max_context": args.max_context if args.max_context is not None else cfg.model.max_context, "max_queue": cfg.serving.max_queue,
                "layer_pipeline": args.partition_policy.startswith("layer_pp") or cfg.parallel.policy == "layer_pp",
                "speculative": (cfg.speculative.mode, cfg.speculative.draft_len),
                "profile": args.serving_profile or None}
    return args, settings


def main(argv=None) -> int:
    args, st = parse_server_args(argv)
    import os
    from . import backends, distributed
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    group = None
    if world > 1:
        # started by torchrun: rank 0 serves HTTP and announces every request, the other ranks follow it
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = distributed.control_group()
    backend, tokenizer = backends.build(st["kind"], args.ckpt, st["max_context"], qwen_dspark=args.qwen_dspark or None,
                                        tokenizer_path=args.tokenizer_path, layer_pipeline=st["layer_pipeline"], speculative=st["speculative"])
    if world > 1 and rank != 0:
        served = distributed.worker_loop(backend, group)
        print(f"worker {rank}: served {served} requests", flush=True)
        return 0
    if world > 1:
        backend = distributed.DistributedBackend(backend, group)
    app = OpenAIApp(ServingEngine(backend, max_queue=st["max_queue"]), tokenizer, model_name=st["model_name"], max_context=st["max_context"])
    httpd = serve(app, st["host"], st["port"])
    print(f"listening on http://{st['host']}:{httpd.server_address[1]} model={st['model_name']} backend={st['kind']} profile={st['profile']}", flush=True)
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    if world > 1:
        backend.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
