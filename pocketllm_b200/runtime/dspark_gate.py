"""Cost-model gate for block drafting (DSpark): decide whether a draft round is worth its
latency and how many draft tokens to verify.

Model: a plain step costs `t_plain`; a round costs `t_draft + t_verify(n)` with
`t_verify(n) = verify_base + verify_per_token * n` and commits 1 + (accepted drafts) tokens.
Per-position match probabilities are calibrated online in confidence buckets. A round is
taken when its expected tokens per second beat plain decoding. Behaviour of the
reference's `DSparkGate` (src/models/deepseek_v4/dspark_gate.py:94-255; cost constants from
docs/dspark.md:19-24 are the defaults for its hardware, here they are constructor inputs and
can be measured with `calibrate_costs`).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class GateCosts:
    plain_ms: float = 303.0
    draft_ms: float = 196.0
    verify_base_ms: float = 300.0
    verify_per_token_ms: float = 109.0


@dataclass
class DSparkGate:
    costs: GateCosts = field(default_factory=GateCosts)
    max_draft: int = 5
    margin_threshold: float = 0.0      # target-logit margin below which drafting is skipped
    n_buckets: int = 10
    prior_match: float = 0.6
    prior_weight: float = 4.0

    def __post_init__(self) -> None:
        # [position][bucket] -> (matches, trials)
        self._cal = [[[self.prior_match * self.prior_weight, self.prior_weight] for _ in range(self.n_buckets)]
                     for _ in range(self.max_draft)]
        self.stats = {"rounds": 0, "drafted": 0, "skipped": 0, "proposed_tokens": 0, "accepted_tokens": 0}

    def _bucket(self, conf: float) -> int:
        return min(self.n_buckets - 1, max(0, int(conf * self.n_buckets)))

    def match_probability(self, position: int, confidence: float) -> float:
        m, t = self._cal[min(position, self.max_draft - 1)][self._bucket(confidence)]
        return m / t

    def expected_tokens(self, confidences: list[float], n: int) -> float:
        """1 bonus token plus the expected accepted prefix length of the first n drafts."""
        e, alive = 1.0, 1.0
        for i in range(n):
            alive *= self.match_probability(i, confidences[i])
            e += alive
        return e

    def round_ms(self, n: int) -> float:
        c = self.costs
        return c.draft_ms + c.verify_base_ms + c.verify_per_token_ms * n

    def choose_draft_len(self, confidences: list[float]) -> int:
        """Draft length with the best expected tokens per ms; 0 means plain decoding wins."""
        best_n, best_rate = 0, 1.0 / self.costs.plain_ms
        for n in range(1, min(self.max_draft, len(confidences)) + 1):
            rate = self.expected_tokens(confidences, n) / self.round_ms(n)
            if rate > best_rate:
                best_n, best_rate = n, rate
        return best_n

    def should_draft(self, target_margin: float | None = None, typical_confidence: float = 0.7) -> bool:
        """Pre-draft decision (before paying for the draft): skip when the target itself is
        unsure, or when even an optimistic round cannot beat plain decoding."""
        if target_margin is not None and target_margin < self.margin_threshold:
            self.stats["skipped"] += 1
            return False
        ok = self.choose_draft_len([typical_confidence] * self.max_draft) > 0
        if not ok:
            self.stats["skipped"] += 1
        return ok

    def observe(self, confidences: list[float], accepted: int, proposed: int) -> None:
        """Update the calibration with one verified round (drafts 0..accepted-1 matched, draft
        `accepted` did not when accepted < proposed)."""
        self.stats["rounds"] += 1
        self.stats["drafted"] += 1
        self.stats["proposed_tokens"] += proposed
        self.stats["accepted_tokens"] += accepted
        for i in range(min(proposed, self.max_draft, len(confidences))):
            if i > accepted:
                break
            cell = self._cal[i][self._bucket(confidences[i])]
            cell[1] += 1.0
            if i < accepted:
                cell[0] += 1.0

    def acceptance_rate(self) -> float:
        p = self.stats["proposed_tokens"]
        return self.stats["accepted_tokens"] / p if p else 0.0
