"""Greedy speculative decoding over an engine with verify rows and state snapshots.

One round: a drafter proposes up to `k` tokens after the last generated token `t0`; the engine
scores the rows `[t0, d1 .. d_{k-1}]` in ONE weight-streaming pass (`forward_rows`, <= 8 rows);
row i predicts the token after it, so drafts are accepted while `pred[i] == d_{i+1}`. With `a`
accepted drafts the round emits `d1..d_a` plus the bonus token `pred[a]`. If some rows were
rejected, the recurrent state (which, unlike the KV cache, cannot be truncated) is rewound to
the snapshot taken before the round and the accepted rows are replayed. Output equals plain
greedy decoding token for token (the reference's contract for its MTP and DSpark loops,
cpp_engine/src/qwen_model.cu:6333-6711, 7160-7710).

Drafters: `NGramDrafter` (prompt lookup, no model), `ReplayDrafter` (a fixed continuation;
used by tests as the perfect or adversarial draft), or anything with `propose(context, k)`.
A gate (`runtime.dspark_gate`) can veto or shorten a round; a vetoed round runs one plain step.
Model-free drafters carry no confidences, so the gate sees `gate_confidence` for every draft.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Protocol, Sequence


class Drafter(Protocol):
    def propose(self, context: Sequence[int], k: int) -> list[int]: ...


class NGramDrafter:
    """Prompt-lookup drafting: find the latest earlier occurrence of the last `n` tokens and
    propose what followed it."""

    def __init__(self, max_ngram: int = 4, min_ngram: int = 1):
        self.max_ngram, self.min_ngram = max_ngram, min_ngram

    def propose(self, context: Sequence[int], k: int) -> list[int]:
        ctx = list(context)
        for n in range(min(self.max_ngram, len(ctx) - 1), self.min_ngram - 1, -1):
            tail = ctx[-n:]
            for start in range(len(ctx) - n - 1, -1, -1):
                if ctx[start:start + n] == tail:
                    cont = ctx[start + n:start + n + k]
                    if cont:
                        return cont
        return []


class ReplayDrafter:
    """Proposes from a known continuation of the generated stream (index 0 = first generated token)."""

    def __init__(self, continuation: Sequence[int], prompt_len: int):
        self.cont, self.prompt_len = list(continuation), prompt_len

    def propose(self, context: Sequence[int], k: int) -> list[int]:
        done = len(context) - self.prompt_len
        return self.cont[done:done + k]


@dataclass
class SpecStats:
    rounds: int = 0
    plain_steps: int = 0
    drafted: int = 0
    accepted: int = 0
    replays: int = 0
    emitted: int = 0
    accept_hist: list[int] = field(default_factory=list)

    @property
    def acceptance(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    @property
    def tokens_per_pass(self) -> float:
        passes = self.rounds + self.plain_steps + self.replays
        return self.emitted / passes if passes else 0.0


def speculative_generate(engine, prompt: Sequence[int], max_new_tokens: int, drafter: Drafter, k: int = 4, *, gate=None,
                         gate_confidence: float = 0.7, eos: int | None = None) -> tuple[list[int], SpecStats]:
    """Returns (generated tokens, stats). `engine` needs prefill / forward_rows / snapshot."""
    if not 1 <= k <= 7:
        raise ValueError("k must be in 1..7 (verify passes hold at most 8 rows)")
    stats = SpecStats()
    out = [engine.prefill(prompt)]
    ctx = list(prompt) + out
    snap = engine.snapshot()
    try:
        while len(out) < max_new_tokens and (eos is None or out[-1] != eos):
            room = max_new_tokens - len(out)
            draft = drafter.propose(ctx, min(k, room - 1)) if room > 1 else []
            if gate is not None and draft:
                conf = [gate_confidence] * len(draft)
                draft = draft[:gate.choose_draft_len(conf)] if gate.should_draft(typical_confidence=gate_confidence) else []
            if not draft:
                nxt = engine.forward_rows([out[-1]])[0]
                stats.plain_steps += 1
                new = [nxt]
            else:
                snap.update()
                rows = [out[-1]] + draft            # k+1 rows: the last one yields the bonus after a full accept
                pred = engine.forward_rows(rows)
                a = 0
                while a < len(draft) and pred[a] == draft[a]:
                    a += 1
                stats.rounds += 1
                stats.drafted += len(draft)
                stats.accepted += a
                stats.accept_hist.append(a)
                if a < len(draft):
                    snap.restore()
                    pred = engine.forward_rows(rows[:a + 1])
                    stats.replays += 1
                new = draft[:a] + [pred[a]]
                if gate is not None:
                    gate.observe([gate_confidence] * len(draft), a, len(draft))
            if eos is not None and eos in new:
                new = new[:new.index(eos) + 1]
            out += new
            ctx += new
            stats.emitted += len(new)
    finally:
        snap.free()
    return out[:max_new_tokens], stats


class DrafterSpeculator:
    """Round-at-a-time form of `speculative_generate` for serving loops: `prefill(prompt)` returns the first token,
    `decode(last, n)` runs ONE round (draft, verify rows, rewind and replay on a reject) and returns between 1 and n new
    tokens. Tokens equal plain greedy decoding. Same interface as the block-drafter speculator of the Qwen backend, so any
    model-free drafter (`NGramDrafter`) can speed up greedy requests."""

    def __init__(self, engine, drafter: Drafter, k: int = 4):
        if not 1 <= k <= 7:
            raise ValueError("k must be in 1..7 (verify passes hold at most 8 rows)")
        self.engine, self.drafter, self.k = engine, drafter, k
        self.ctx: list[int] = []
        self.snap = None
        self.stats = SpecStats()

    def prefill(self, prompt: Sequence[int]) -> int:
        first = self.engine.prefill(list(prompt))
        self.ctx = list(prompt) + [first]
        if self.snap is not None:
            self.snap.free()
        self.snap = self.engine.snapshot()
        return first

    def decode(self, last: int, n: int) -> list[int]:
        if n < 1:
            return []
        draft = self.drafter.propose(self.ctx, min(self.k, n - 1)) if n > 1 else []
        if not draft:
            new = [self.engine.forward_rows([last])[0]]
            self.stats.plain_steps += 1
        else:
            self.snap.update()
            rows = [last] + draft
            pred = self.engine.forward_rows(rows)
            a = 0
            while a < len(draft) and pred[a] == draft[a]:
                a += 1
            self.stats.rounds += 1
            self.stats.drafted += len(draft)
            self.stats.accepted += a
            self.stats.accept_hist.append(a)
            if a < len(draft):
                self.snap.restore()
                pred = self.engine.forward_rows(rows[:a + 1])
                self.stats.replays += 1
            new = draft[:a] + [pred[a]]
        self.ctx += new
        self.stats.emitted += len(new)
        return new
