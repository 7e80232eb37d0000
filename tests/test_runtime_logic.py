"""Pure-CPU runtime logic: prefix snapshot cache, PD scheduler, DSpark gate."""
from pocketllm_b200.runtime.dspark_gate import DSparkGate, GateCosts
from pocketllm_b200.runtime.pd_scheduler import PDScheduler, PhaseResources
from pocketllm_b200.runtime.prefix_snapshot import PrefixSnapshotCache, chain_hashes


def test_chain_hashes_are_prefix_stable():
    a = list(range(600))
    b = a[:512] + [7] * 88
    ha, hb = chain_hashes(a), chain_hashes(b)
    assert len(ha) == 2 and ha == hb                       # same first 512 tokens
    assert chain_hashes(a[:255]) == [] and chain_hashes([1] + a[1:600])[0] != ha[0]


def test_prefix_cache_restore_capture_lru():
    evicted = []
    c = PrefixSnapshotCache(capacity=2, on_evict=lambda s: evicted.append(s.length))
    p = list(range(1000))
    assert c.restore(p) is None
    assert c.capture(p[:256], "s256") and c.capture(p[:512], "s512")
    assert c.lookup_hint(p) == 512
    assert c.restore(p).state == "s512"
    assert c.restore(p[:512]).state == "s256"              # must leave one token to compute
    assert c.restore(p[:256]) is None
    q = [5] * 300
    c.capture(q, "q256")                                    # evicts the least recently used
    assert len(c) == 2 and evicted == [512]
    assert c.restore([1] + p[1:]) is None and c.stats["hits"] == 2
    assert not c.capture([1, 2, 3], "short")


def test_pd_scheduler_prefers_decode():
    s = PDScheduler(prefill=PhaseResources(env={"POCKET_PHASE": "prefill"}), decode=PhaseResources(env={"POCKET_PHASE": "decode"}),
                    max_pending=3)
    assert s.submit("a") and s.submit("b")
    req, phase = s.next()
    assert (req, phase) == ("a", "prefill")
    s.prefill_done("a")
    assert s.next() == ("a", "decode")                      # decode before the second prefill
    s.requeue_decode("a")
    assert s.next() == ("a", "decode")
    assert s.next() == ("b", "prefill")
    assert s.next(timeout=0.01) is None
    assert s.submit("c") and s.submit("d") and s.submit("e") and not s.submit("f")
    assert s.stats["rejected"] == 1 and s.stats["phase_switches"] >= 3
    import os
    assert os.environ["POCKET_PHASE"] == "prefill"


def test_dspark_gate_decisions_and_calibration():
    g = DSparkGate(GateCosts(plain_ms=300, draft_ms=200, verify_base_ms=300, verify_per_token_ms=100), max_draft=5)
    # with the 0.6 prior a round (>= 600 ms) cannot beat 300 ms per token
    assert g.choose_draft_len([0.9] * 5) == 0 and not g.should_draft()
    for _ in range(200):
        g.observe([0.95] * 5, accepted=5, proposed=5)
    assert g.match_probability(0, 0.95) > 0.95
    n = g.choose_draft_len([0.95] * 5)
    assert n == 5 and g.expected_tokens([0.95] * 5, 5) > 5.0
    # low-confidence buckets stay at the prior and are rejected
    assert g.choose_draft_len([0.1] * 5) == 0
    assert abs(g.acceptance_rate() - 1.0) < 1e-9
    g2 = DSparkGate(GateCosts(300, 20, 30, 10), margin_threshold=0.5)
    assert not g2.should_draft(target_margin=0.1) and g2.should_draft(target_margin=2.0)
    g2.observe([0.5, 0.5, 0.5], accepted=1, proposed=3)
    assert g2.stats["accepted_tokens"] == 1 and g2.stats["proposed_tokens"] == 3


# ---------------------------------------------------------------------------------------
# speculative loop against a fake engine (deterministic next-token function + recurrent state)
class _FakeSnap:
    def __init__(self, e):
        self.e, self.state = e, None
        self.update()

    def update(self):
        self.state = (self.e.h, self.e.pos)

    def restore(self):
        self.e.h, self.e.pos = self.state

    def free(self):
        pass


class _FakeEngine:
    """next token = f(running hash of all tokens fed so far): any wrong rewind changes the output."""

    def __init__(self):
        self.h, self.pos, self.passes = 0, 0, 0

    def _feed(self, t):
        self.h = (self.h * 1000003 + t + 1) % 2147483647
        self.pos += 1
        return (self.h >> 3) % 11      # small vocabulary so that n-grams repeat

    def prefill(self, prompt):
        self.h, self.pos = 0, 0
        for t in prompt:
            nxt = self._feed(t)
        return nxt

    def forward_rows(self, rows):
        assert 1 <= len(rows) <= 8
        self.passes += 1
        return [self._feed(t) for t in rows]

    def snapshot(self):
        return _FakeSnap(self)


def _plain(prompt, n):
    e = _FakeEngine()
    out = [e.prefill(prompt)]
    while len(out) < n:
        out.append(e.forward_rows([out[-1]])[0])
    return out


def test_speculative_matches_plain_greedy_for_any_drafter():
    from pocketllm_b200.runtime.speculative import NGramDrafter, ReplayDrafter, speculative_generate
    prompt = [1, 2, 3, 4, 5, 1, 2, 3]
    ref = _plain(prompt, 40)
    # perfect draft: every round accepts k and emits k+1
    e = _FakeEngine()
    out, st = speculative_generate(e, prompt, 40, ReplayDrafter(ref[1:] , len(prompt) + 1), k=4)
    assert out == ref and st.acceptance == 1.0 and st.replays == 0 and st.tokens_per_pass > 4.0
    # adversarial draft: always wrong -> one replay per round, still identical output
    bad = [(t + 1) % 11 for t in ref[1:]]
    out, st = speculative_generate(_FakeEngine(), prompt, 40, ReplayDrafter(bad, len(prompt) + 1), k=3)
    assert out == ref and st.accepted == 0 and st.replays == st.rounds
    # half-right draft: rewinds in the middle of a round
    half = [t if i % 3 else (t + 5) % 11 for i, t in enumerate(ref[1:])]
    out, st = speculative_generate(_FakeEngine(), prompt, 40, ReplayDrafter(half, len(prompt) + 1), k=5)
    assert out == ref and 0 < st.acceptance < 1
    out, st = speculative_generate(_FakeEngine(), prompt, 40, NGramDrafter(), k=4)
    assert out == ref


def test_round_at_a_time_speculator_matches_plain_greedy():
    from pocketllm_b200.runtime.speculative import DrafterSpeculator, NGramDrafter, ReplayDrafter
    prompt = [1, 2, 3, 4, 5, 1, 2, 3]
    ref = _plain(prompt, 40)
    for drafter in (NGramDrafter(), ReplayDrafter(ref[1:], len(prompt) + 1), ReplayDrafter([(t + 1) % 11 for t in ref[1:]], len(prompt) + 1)):
        sp = DrafterSpeculator(_FakeEngine(), drafter, k=4)
        out = [sp.prefill(prompt)]
        while len(out) < 40:
            new = sp.decode(out[-1], min(8, 40 - len(out)))
            assert 1 <= len(new) <= min(8, 40 - len(out))
            out += new
        assert out == ref
    assert sp.stats.replays == sp.stats.rounds > 0                     # the adversarial drafter: every round rewinds
    # a second request on the same speculator starts from a fresh context
    assert sp.prefill(prompt) == ref[0] and sp.ctx == prompt + [ref[0]]


def test_speculative_respects_eos_and_gate():
    from pocketllm_b200.runtime.dspark_gate import DSparkGate
    from pocketllm_b200.runtime.speculative import ReplayDrafter, speculative_generate
    prompt = [4, 4, 2]
    ref = _plain(prompt, 30)
    eos = ref[7]
    cut = ref[:ref.index(eos) + 1]
    out, _ = speculative_generate(_FakeEngine(), prompt, 30, ReplayDrafter(ref[1:], len(prompt) + 1), k=4, eos=eos)
    assert out == cut
    gate = DSparkGate()
    out, st = speculative_generate(_FakeEngine(), prompt, 30, ReplayDrafter(ref[1:], len(prompt) + 1), k=4, gate=gate)
    assert out == ref and gate.stats["rounds"] == st.rounds


def test_lru_slots_and_waves():
    import torch
    from pocketllm_b200.moe.expert_cache import LRUSlots, waves
    lru = LRUSlots(3)
    m, copies = lru.assign([5, 1, 5])
    assert set(m) == {5, 1} and len(copies) == 2 and lru.stats == {"hits": 0, "misses": 2, "evictions": 0}
    m, copies = lru.assign([7])
    assert len(copies) == 1 and lru.stats["evictions"] == 0
    m, copies = lru.assign([1, 9])                          # 5 is the least recently used and goes
    assert copies == [(9, m[9])] and 5 not in lru.where and lru.stats["evictions"] == 1 and lru.stats["hits"] == 1
    m, copies = lru.assign([5, 7, 9])                       # 1 must go although it was used more recently than 7's slot holder
    assert 1 not in lru.where and len({m[5], m[7], m[9]}) == 3
    import pytest
    with pytest.raises(ValueError):
        lru.assign([0, 1, 2, 3])
    ids = torch.tensor([[0, 1], [1, 2], [3, 4], [4, 0], [5, 6]])
    assert waves(ids, 3) == [(0, 2), (2, 4), (4, 5)]
    assert waves(ids, 8) == [(0, 5)]


def test_expert_slots_planned_from_a_memory_budget():
    from pocketllm_b200.moe.expert_cache import slots_for_budget
    gib = 1 << 30
    # 40 layers of 256 experts at 20 MiB each = 200 GiB: 100 GiB hold half of them
    assert slots_for_budget(100 * gib, 20 << 20, 40, 256, 8) == 128
    assert slots_for_budget(400 * gib, 20 << 20, 40, 256, 8) is None          # everything fits: no staging
    assert slots_for_budget(1 * gib, 20 << 20, 40, 256, 8) == 9                # never below one token's experts plus a prefetch slot
    assert slots_for_budget(0, 20 << 20, 40, 4, 8) == 4                        # ... nor above the expert count
    import pytest
    with pytest.raises(ValueError):
        slots_for_budget(gib, 0, 40, 256, 8)


def test_gate_overlap_analysis_of_a_router_dump(tmp_path):
    import json
    import torch
    from pocketllm_b200.moe import analyze_gate_overlap as ago
    # layer 0 repeats its experts from token to token, layer 1 never does
    capture = {"layers.0.ffn.route_idx": [torch.tensor([[0, 1], [0, 1], [0, 2]]), torch.tensor([[0, 2]]), torch.tensor([[0, 2]])],
               "layers.1.ffn.route_idx": [torch.tensor([[0, 1], [2, 3], [4, 5]]), torch.tensor([[6, 7]]), torch.tensor([[0, 1]])],
               "layers.0.attn.index_sel": [[1, 2]]}
    path = tmp_path / "dump.jsonl"
    assert ago.dump_capture(capture, path) == 6
    first = json.loads(path.read_text().splitlines()[0])
    assert first == {"layer": 0, "ids": [[0, 1], [0, 1], [0, 2]]}
    with open(path) as f:
        res = ago.analyze(f, [2, 4])
    assert res["0"]["tokens"] == 5 and res["0"]["distinct_experts"] == 3
    assert res["0"]["mean_consecutive_overlap"] == (1.0 + 0.5 + 1.0 + 1.0) / 4
    assert res["1"]["mean_consecutive_overlap"] == 0.0 and res["1"]["lru_hit_rate"]["2"] == 0.0
    # layer 0 with 4 slots: 3 cold misses out of 10 uses
    assert abs(res["0"]["lru_hit_rate"]["4"] - 0.7) < 1e-9
    with open(path) as f:
        dec = ago.analyze(f, [1], skip_prefill=True)
    assert dec["0"]["tokens"] == 3 and dec["0"]["lru_hit_rate"]["1"] is None      # two experts per token do not fit one slot
    assert ago.main([str(path), "--slots", "2,4"]) == 0
