"""Sidecar of the native OpenAI server (`pocket_engine --serve`): chat templating, tokenisation,
incremental detokenisation with stop strings, and parsing of the finished completion. One JSON
object per line on stdin, one reply per line on stdout (role of the reference's
cpp_engine/tools/cpp_sidecar.py).

    {"op": "hello"}                      -> {"ok": true, "eos": [...]}
    {"op": "begin", "body": <request>}   -> {"ok": true, "tokens": [...], "max_tokens": N, "stop_token_ids": [...],
                                             "stream": b, "temperature": t, "top_p": p, "top_k": k, "min_p": m, "frequency_penalty": f,
                                             "presence_penalty": q, "repetition_penalty": r, "seed": s,
                                             "include_usage": b}   |  {"ok": false, "status": 400, "error": "..."}
    {"op": "token", "token": id}         -> {"delta": "text", "channel": "content" | "reasoning_content", "stop": b}
    {"op": "end", "finish_reason": r}    -> {"tail": "text", "channel": ..., "message": {...}, "finish_reason": r'}
    {"op": "token_texts", "ids": [...]}  -> {"texts": [...]}    (the text of single tokens, for log-probability reports)
    {"op": "quit"}
"""
from __future__ import annotations

import argparse
import json
import sys

from ..encoding import dsv4
from .openai import BadRequest, StreamingDecoder, build_params, with_tool_directive


class CharTokenizer:
    """One token per character (id = code point, 0 = EOS) with the DSV4 chat framing; for tests."""
    eos_ids = (0,)

    def __init__(self, chat_format: str = "dsv4"):
        self.chat_format = chat_format

    def encode_chat(self, messages, *, tools=None, thinking=False, reasoning_effort=None, response_format=None):
        if self.chat_format == "plain":                    # ASCII only: for models with a tiny vocabulary
            return [ord(c) for c in "".join(f"{m['role']}: {dsv4._text(m.get('content'))}\n" for m in messages) + "assistant: "]
        text = dsv4.encode_messages(messages, tools=tools, thinking_mode="thinking" if thinking else "chat",
                                    reasoning_effort=reasoning_effort, response_format=response_format)
        return [ord(c) for c in text]

    def decode(self, ids):
        return "".join(chr(i) for i in ids)

    def parse(self, text, thinking):
        return dsv4.parse_completion(("<think>" if thinking else "") + text, "thinking" if thinking else "chat")


def build_tokenizer(spec: str, chat_format: str):
    if spec == "chars":
        return CharTokenizer(chat_format)
    from . import backends
    kind, _, path = spec.partition(":")
    if kind in ("hf", "gguf"):
        return backends.build_tokenizer(kind, path, chat_format)
    raise SystemExit(f"unknown tokenizer spec {spec!r} (chars | hf:DIR | gguf:FILE)")


class Session:
    def __init__(self, tok):
        self.tok = tok
        self.dec: StreamingDecoder | None = None
        self.thinking = False
        self.in_reasoning = False
        self.carry = ""

    def begin(self, body: dict) -> dict:
        try:
            p, opts = build_params(body, tuple(self.tok.eos_ids))
            if opts["n"] != 1:
                raise BadRequest("the native server generates one choice per request")
            messages = with_tool_directive(body["messages"], opts["tools"], body.get("tool_choice"), body.get("parallel_tool_calls"))
            ids = self.tok.encode_chat(messages, tools=opts["tools"], thinking=opts["thinking"],
                                       reasoning_effort=opts["reasoning_effort"], response_format=opts["response_format"])
        except BadRequest as e:
            return {"ok": False, "status": 400, "error": str(e)}
        except Exception as e:                                   # malformed messages and the like
            return {"ok": False, "status": 400, "error": f"could not encode the conversation: {e}"}
        self.dec = StreamingDecoder(self.tok, opts["stop"])
        self.thinking = self.in_reasoning = bool(opts["thinking"])
        self.carry = ""
        return {"ok": True, "tokens": [int(t) for t in ids], "max_tokens": p.max_tokens, "stop_token_ids": list(p.stop_token_ids),
                "stream": opts["stream"], "temperature": p.temperature, "top_p": p.top_p, "top_k": p.top_k, "min_p": p.min_p,
                "frequency_penalty": p.frequency_penalty, "presence_penalty": p.presence_penalty, "repetition_penalty": p.repetition_penalty,
                "seed": int(p.seed or 0), "include_usage": opts["include_usage"], "logprobs": p.logprobs}

    def _split(self, text: str, final: bool = False) -> tuple[str, str]:
        """Route a delta to the reasoning or the content channel. While reasoning, text that could still
        grow into the closing tag is held back; the tag itself is never emitted."""
        text = self.carry + text
        self.carry = ""
        if not self.in_reasoning:
            return "content", text
        tag = dsv4.THINK_CLOSE
        if tag in text:
            self.in_reasoning = False
            head, rest = text.split(tag, 1)
            if head or final:
                self.carry = rest                    # content that arrived with the tag goes out with the next delta
                return "reasoning_content", head
            return "content", rest
        hold = 0 if final else next((k for k in range(min(len(tag) - 1, len(text)), 0, -1) if text.endswith(tag[:k])), 0)
        if hold:
            self.carry = text[-hold:]
            text = text[:-hold]
        return "reasoning_content", text

    def token(self, t: int) -> dict:
        delta = self.dec.push(int(t))
        ch, delta = self._split(delta)
        return {"delta": delta, "channel": ch, "stop": self.dec.stopped}

    def end(self, finish: str) -> dict:
        tail = self.dec.flush()
        ch, tail = self._split(tail, final=True)
        if self.carry:                                   # content held back behind a closing tag in the last delta
            ch, tail = ("content", self.carry) if not tail else (ch, tail)
            self.carry = ""
        msg = self.tok.parse(self.dec.text, self.thinking)
        if msg.get("tool_calls"):
            finish = "tool_calls"
        return {"tail": tail, "channel": ch, "message": msg, "finish_reason": finish}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokenizer", default="chars")
    ap.add_argument("--chat-format", default="dsv4")
    args = ap.parse_args(argv)
    s = Session(build_tokenizer(args.tokenizer, args.chat_format))
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        req = json.loads(line)
        op = req.get("op")
        if op == "quit":
            break
        if op == "hello":
            out = {"ok": True, "eos": list(s.tok.eos_ids)}
        elif op == "begin":
            out = s.begin(req.get("body") or {})
        elif op == "token":
            out = s.token(req["token"])
        elif op == "end":
            out = s.end(req.get("finish_reason", "stop"))
        elif op == "token_texts":
            out = {"texts": [s.tok.decode([int(i)]) for i in req.get("ids", [])]}
        else:
            out = {"ok": False, "status": 400, "error": f"unknown op {op!r}"}
        sys.stdout.write(json.dumps(out, ensure_ascii=False) + "\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
