"""DeepSeek-V4 chat framing: prompt rendering (system / user / assistant / tool turns,
thinking modes, reasoning effort, tool schemas and tool calls in the DSML markup) and the
inverse, parsing a completion into content, reasoning and tool calls.

Wire format (what the model was trained on; reference implementation:
src/encoding/dsv4.py:20-119 constants, 242-423 message rendering, 656-760 parsing):

    <BOS>{system}<｜User｜>{user}<｜Assistant｜><think>{reasoning}</think>{content}{tool calls}<EOS>

* thinking mode "chat": the assistant turn opens with `</think>` (no reasoning);
  "thinking": it opens with `<think>`; reasoning of turns before the last user message is
  dropped and rendered as a bare `</think>`.
* tool calls: `<｜DSML｜tool_calls>` block of `<｜DSML｜invoke name="f">` elements whose
  `<｜DSML｜parameter name="k" string="true|false">v</｜DSML｜parameter>` children carry strings
  verbatim and everything else as JSON. Tool results come back inside the next user turn as
  `<tool_result>...</tool_result>`.
"""
from __future__ import annotations

import json
import re
from typing import Any

BOS = "<｜begin▁of▁sentence｜>"
EOS = "<｜end▁of▁sentence｜>"
USER = "<｜User｜>"
ASSISTANT = "<｜Assistant｜>"
THINK_OPEN, THINK_CLOSE = "<think>", "</think>"
DSML = "｜DSML｜"

REASONING_EFFORT_PROMPTS = {
    "low": "",
    "high": ("Reasoning Effort: Absolute maximum with no shortcuts permitted.\n"
             "You MUST be very thorough in your thinking and comprehensively decompose the problem to resolve the root cause, "
             "rigorously stress-testing your logic against all potential paths, edge cases, and adversarial scenarios.\n"
             "Explicitly write out your entire deliberation process, documenting every intermediate step, considered alternative, "
             "and rejected hypothesis to ensure absolutely no assumption is left unchecked.\n\n"),
    "max": ("Reasoning Effort: Beyond maximum — exhaustive, relentless, and uncompromising.\n"
            "You MUST reason with the utmost depth and rigor, leaving absolutely nothing to chance: exhaustively decompose the problem "
            "into its most fundamental components, trace every causal chain to its root, and resolve the underlying cause rather than "
            "any surface symptom.\n"
            "Do not stop reasoning until you have independently verified the solution from multiple angles and are certain that no "
            "assumption remains unchecked and no error remains undiscovered.\n\n"),
}
EFFORT_ALIASES = {"minimal": "low", "medium": "low"}


def _json(v: Any) -> str:
    return json.dumps(v, ensure_ascii=False)


def normalize_effort(effort: str | None) -> str:
    e = (effort or "low").lower()
    e = EFFORT_ALIASES.get(e, e)
    if e not in REASONING_EFFORT_PROMPTS:
        raise ValueError(f"unknown reasoning effort {effort!r}")
    return e


def render_tools(tools: list[dict]) -> str:
    """System-prompt section that teaches the DSML call syntax and lists the schemas."""
    schemas = "\n".join(_json(t.get("function", t)) for t in tools)
    return (
        "## Tools\n\n"
        "You have access to a set of tools to help answer the user's question. You can invoke tools by writing a "
        f"\"<{DSML}tool_calls>\" block like the following:\n\n"
        f"<{DSML}tool_calls>\n<{DSML}invoke name=\"$TOOL_NAME\">\n"
        f"<{DSML}parameter name=\"$PARAMETER_NAME\" string=\"true|false\">$PARAMETER_VALUE</{DSML}parameter>\n...\n"
        f"</{DSML}invoke>\n<{DSML}invoke name=\"$TOOL_NAME2\">\n...\n</{DSML}invoke>\n</{DSML}tool_calls>\n\n"
        "String parameters should be specified as is and set `string=\"true\"`. For all other types (numbers, booleans, arrays, "
        "objects), pass the value in JSON format and set `string=\"false\"`.\n\n"
        f"If thinking_mode is enabled (triggered by {THINK_OPEN}), you MUST output your complete reasoning inside "
        f"{THINK_OPEN}...{THINK_CLOSE} BEFORE any tool calls or final response.\n\n"
        f"Otherwise, output directly after {THINK_CLOSE} with tool calls or final response.\n\n"
        f"### Available Tool Schemas\n\n{schemas}\n\n"
        "You MUST strictly follow the above defined tool name and parameter schemas to invoke tool calls.\n")


def render_tool_calls(tool_calls: list[dict]) -> str:
    """OpenAI-style tool calls -> DSML block."""
    blocks = []
    for tc in tool_calls:
        fn = tc.get("function", tc)
        args = fn.get("arguments", "{}")
        try:
            args = json.loads(args) if isinstance(args, str) else dict(args)
        except Exception:
            args = {"arguments": args}
        params = "\n".join(
            f"<{DSML}parameter name=\"{k}\" string=\"{'true' if isinstance(v, str) else 'false'}\">"
            f"{v if isinstance(v, str) else _json(v)}</{DSML}parameter>" for k, v in args.items())
        blocks.append(f"<{DSML}invoke name=\"{fn['name']}\">\n{params}\n</{DSML}invoke>")
    return f"<{DSML}tool_calls>\n" + "\n".join(blocks) + f"\n</{DSML}tool_calls>"


def _text(content: Any) -> str:
    """OpenAI content may be a string or a list of {type: text} blocks."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    return "".join(b.get("text", "") for b in content if isinstance(b, dict) and b.get("type") in (None, "text", "input_text"))


def merge_tool_messages(messages: list[dict]) -> list[dict]:
    """Fold `tool` role messages into a user turn of <tool_result> blocks, in call order."""
    out: list[dict] = []
    for m in messages:
        if m.get("role") == "tool":
            block = f"<tool_result>{_text(m.get('content'))}</tool_result>"
            if out and out[-1].get("role") == "user" and out[-1].get("_tool_results"):
                out[-1]["content"] += "\n\n" + block
            else:
                out.append({"role": "user", "content": block, "_tool_results": True})
        else:
            out.append(dict(m))
    return out


def encode_messages(messages: list[dict], *, thinking_mode: str = "chat", tools: list[dict] | None = None,
                    reasoning_effort: str | None = None, response_format: dict | None = None,
                    add_generation_prompt: bool = True, drop_thinking: bool = True) -> str:
    """Render a conversation to the prompt string the model continues."""
    if thinking_mode not in ("chat", "thinking"):
        raise ValueError("thinking_mode must be 'chat' or 'thinking'")
    msgs = merge_tool_messages(messages)
    last_user = max((i for i, m in enumerate(msgs) if m.get("role") in ("user", "developer")), default=-1)
    out = BOS
    if thinking_mode == "thinking":
        out += REASONING_EFFORT_PROMPTS[normalize_effort(reasoning_effort)]
    system_parts = [_text(m.get("content")) for m in msgs if m.get("role") == "system"]
    if tools:
        system_parts.append(render_tools(tools))
    if response_format and response_format.get("type") in ("json_object", "json_schema"):
        schema = response_format.get("json_schema", {}).get("schema", {"type": "object"})
        system_parts.append("## Response Format:\n\nYou MUST strictly adhere to the following schema to reply:\n" + _json(schema))
    out += "\n\n".join(p for p in system_parts if p)
    for i, m in enumerate(msgs):
        role = m.get("role")
        if role == "system":
            continue
        if role in ("user", "developer"):
            out += USER + _text(m.get("content"))
        elif role == "assistant":
            reasoning = m.get("reasoning_content") or ""
            keep = thinking_mode == "thinking" and reasoning and not (drop_thinking and i < last_user)
            out += ASSISTANT + ((THINK_OPEN + reasoning + THINK_CLOSE) if keep else THINK_CLOSE)
            out += _text(m.get("content"))
            if m.get("tool_calls"):
                out += "\n\n" + render_tool_calls(m["tool_calls"])
            out += EOS
        else:
            raise ValueError(f"unknown role {role!r}")
    if add_generation_prompt and (not msgs or msgs[-1].get("role") != "assistant"):
        out += ASSISTANT + (THINK_OPEN if thinking_mode == "thinking" else THINK_CLOSE)
    return out


_INVOKE_RE = re.compile(rf"<{DSML}invoke name=\"(?P<name>[^\"]+)\">\s*(?P<body>.*?)\s*</{DSML}invoke>", re.S)
_PARAM_RE = re.compile(rf"<{DSML}parameter name=\"(?P<k>[^\"]+)\" string=\"(?P<s>true|false)\">(?P<v>.*?)</{DSML}parameter>", re.S)


def parse_tool_calls(text: str) -> tuple[str, list[dict]]:
    """Split `text` into (content before the DSML block, OpenAI-style tool calls)."""
    start = text.find(f"<{DSML}tool_calls>")
    if start < 0:
        return text, []
    end = text.find(f"</{DSML}tool_calls>", start)
    block = text[start: end if end >= 0 else len(text)]
    calls = []
    for n, m in enumerate(_INVOKE_RE.finditer(block)):
        args: dict[str, Any] = {}
        for pm in _PARAM_RE.finditer(m.group("body")):
            v = pm.group("v")
            if pm.group("s") == "false":
                try:
                    v = json.loads(v)
                except Exception:
                    pass
            args[pm.group("k")] = v
        calls.append({"id": f"call_{n}", "type": "function", "function": {"name": m.group("name"), "arguments": _json(args)}})
    return text[:start].rstrip(), calls


def parse_completion(text: str, thinking_mode: str = "chat") -> dict:
    """Completion text (after the generation prompt) -> assistant message dict."""
    text = text.split(EOS, 1)[0]
    reasoning = ""
    if thinking_mode == "thinking":
        if THINK_CLOSE in text:
            reasoning, text = text.split(THINK_CLOSE, 1)
            reasoning = reasoning.replace(THINK_OPEN, "", 1)
        else:
            reasoning, text = text.replace(THINK_OPEN, "", 1), ""
    elif text.startswith(THINK_CLOSE):
        text = text[len(THINK_CLOSE):]
    content, calls = parse_tool_calls(text)
    msg: dict[str, Any] = {"role": "assistant", "content": content}
    if reasoning:
        msg["reasoning_content"] = reasoning
    if calls:
        msg["tool_calls"] = calls
    return msg
