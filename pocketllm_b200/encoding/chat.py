"""Compact chat framing of the GGUF model families (system / user / assistant turns for
raw-token generation; the full Jinja templates travel in the GGUF metadata).

GLM-DSA:   `[gMASK]<sop>` then `<|system|>\\n..`, `<|user|>\\n..`, `<|assistant|>` (+ `\\n<think>`)
MiniMax-M2: `]~!b[]~b]system\\n..[e~[\\n]~b]user\\n..[e~[\\n]~b]ai\\n` (+ `<think>\\n`)
(reference: src/encoding/glm_dsa.py:30-55, src/encoding/minimax_m2.py:30-60)
"""
from __future__ import annotations

GLM_DEFAULT_SYSTEM = "You are a helpful assistant."
MINIMAX_DEFAULT_SYSTEM = "You are a helpful assistant. Your name is MiniMax-M2.7 and is built by MiniMax."


def render_glm(messages: list[dict] | str, *, system_prompt: str | None = None, thinking: bool = False) -> str:
    msgs = [{"role": "user", "content": messages}] if isinstance(messages, str) else list(messages)
    out = "[gMASK]<sop>"
    if system_prompt and not any(m["role"] == "system" for m in msgs):
        out += "<|system|>\n" + system_prompt
    for m in msgs:
        role = m["role"]
        if role not in ("system", "user", "assistant", "observation"):
            raise ValueError(f"unknown role {role!r}")
        out += f"<|{role}|>\n{m.get('content') or ''}"
    out += "<|assistant|>"
    if thinking:
        out += "\n<think>"
    return out


def render_minimax(messages: list[dict] | str, *, system_prompt: str = MINIMAX_DEFAULT_SYSTEM, thinking: bool = False) -> str:
    msgs = [{"role": "user", "content": messages}] if isinstance(messages, str) else list(messages)
    if not any(m["role"] == "system" for m in msgs):
        msgs = [{"role": "system", "content": system_prompt}] + msgs
    names = {"system": "system", "user": "user", "assistant": "ai", "tool": "tool"}
    out = "]~!b["
    for m in msgs:
        out += f"]~b]{names[m['role']]}\n{m.get('content') or ''}[e~[\n"
    out += "]~b]ai\n"
    if thinking:
        out += "<think>\n"
    return out


def split_thinking(text: str) -> tuple[str, str]:
    """(reasoning, visible) of a completion that may contain a <think>...</think> span."""
    if "</think>" in text:
        r, v = text.split("</think>", 1)
        return r.replace("<think>", "", 1).strip("\n"), v.lstrip("\n")
    return "", text
