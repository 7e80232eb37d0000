"""Tiny end-to-end model: native engine vs the fp32 PyTorch oracle (same idea as the
reference's cpp_engine/tests/test_qwen_engine.cpp:1-110, with random instead of zero weights)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    tensors = qh.random_checkpoint(cfg, seed=1, sigma=0.05)
    d = tmp_path_factory.mktemp("tiny_qwen")
    qh.save_checkpoint(d, cfg, tensors)
    return cfg, tensors, d


def _close(a, b, tol):
    return ((a - b).norm() / b.norm()).item() < tol


def test_engine_matches_oracle_decode_path(tiny):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    ref = qh.ReferenceModel(cfg, tensors)
    prompt = [5, 17, 300, 44, 9, 1000, 2]
    ref_tokens, ref_logits = ref.generate(prompt, 6)
    eng = qh.QwenEngine(cfg, max_context=256, prefill_chunk=64, use_cuda_graph=False).load(d)
    first = eng.prefill(prompt)                      # 7 rows -> weight-streaming path
    assert _close(eng.logits(0), ref_logits[0], 3e-2)
    assert first == ref_tokens[0]
    rest = eng.decode(5)
    assert [first] + rest == ref_tokens
    assert eng.comm_status() == 0
    eng.close()


@pytest.mark.parametrize("shape", ["tiny", "mid"])
def test_persistent_decode_kernel_matches_per_projection_launches(tiny, shape, monkeypatch):
    """One persistent kernel per token against one launch per projection, step by step from the same prompt: close
    logits at every step (so the DeltaNet state, the conv tails and the KV cache evolve alike) and the same greedy
    tokens up to a near-tie."""
    from pocketllm_b200.models import qwen_hybrid as qh
    if shape == "tiny":
        cfg, _, d = tiny
        make = lambda: qh.QwenEngine(cfg, max_context=512, prefill_chunk=64).load(d)
    else:
        cfg = qh.QwenHybridConfig(vocab_size=4096, hidden_size=1024, intermediate_size=3072, num_hidden_layers=8,
                                  num_attention_heads=8, num_key_value_heads=2, linear_num_key_heads=4,
                                  linear_num_value_heads=8, max_position_embeddings=4096)
        make = lambda: qh.QwenEngine(cfg, max_context=512, prefill_chunk=64).init_random(seed=5, sigma=0.05)
    torch.manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (150,)).tolist()
    steps = 24
    runs = []
    for mode in ("0", "1"):
        monkeypatch.setenv("POCKET_DECODE_PERSISTENT", mode)
        eng = make()
        toks, lgs = [eng.prefill(prompt)], []
        for _ in range(steps):
            toks += eng.decode(1)
            lgs.append(eng.logits(0))
        assert eng.persistent_decode == (mode == "1")
        assert eng.comm_status() == 0
        runs.append((toks, lgs))
        eng.close()
    (t0, l0), (t1, l1) = runs
    assert t0[0] == t1[0], (t0, t1)                  # the prefill is the same code in both runs
    for i in range(steps):
        # same inputs so far: the logits must be close; the picks may differ only on a near-tie (the two paths add
        # partial sums in different orders, and a flipped bf16 rounding moves the logits by a few 1e-3)
        assert _close(l1[i], l0[i], 3e-2), i
        if t0[i + 1] != t1[i + 1]:
            top = l0[i].topk(2).values
            assert (top[0] - top[1]).item() < 0.02 * l0[i].abs().max().item(), (i, t0, t1)
            break


def test_cuda_graph_decode_equals_eager(tiny):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    prompt = list(range(3, 40))
    outs = []
    for graph in (False, True):
        eng = qh.QwenEngine(cfg, max_context=256, prefill_chunk=64, use_cuda_graph=graph).load(d)
        outs.append(eng.generate(prompt, 12))
        t = eng.timings()
        assert t["kernel_launches"] > 0
        eng.close()
    assert outs[0] == outs[1]


def test_tensor_core_prefill_matches_streaming_prefill(tiny):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    torch.manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (100,)).tolist()
    big = qh.QwenEngine(cfg, max_context=512, prefill_chunk=64).load(d)      # 64 + 36 rows: tcgen05 GEMMs
    small = qh.QwenEngine(cfg, max_context=512, prefill_chunk=8).load(d)     # 8-row groups: matvec path
    tb, ts = big.prefill(prompt), small.prefill(prompt)
    lb, ls = big.logits(0), small.logits(0)
    assert _close(lb, ls, 3e-2)
    assert big.comm_status() == 0
    if (ls.topk(2).values[0] - ls.topk(2).values[1]) > 0.05 * ls.abs().max():
        assert tb == ts
    # continuing from either state gives the same greedy continuation
    assert big.position == small.position == 100
    big.close()
    small.close()


@pytest.mark.parametrize("mode,tol", [("fp8x2", 3e-2), ("fp8", 2.5e-1), ("shadow", 3e-2), ("umma", 3e-2)])
def test_prefill_gemm_modes_agree_with_streaming_prefill(tiny, mode, tol):
    """Every many-row GEMM of the engine against the eight-row weight-streaming path. The native FP8 modes keep no bf16
    copy of the weights; with two E4M3 terms per activation they stay inside the band of the bf16 modes."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    torch.manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (150,)).tolist()
    big = qh.QwenEngine(cfg, max_context=512, prefill_chunk=128, prefill_gemm=mode).load(d)
    small = qh.QwenEngine(cfg, max_context=512, prefill_chunk=8).load(d)
    assert big.prefill_gemm == mode
    assert (big.prefill_shadow_bytes > 0) == (mode == "shadow")
    tb, ts = big.prefill(prompt), small.prefill(prompt)
    lb, ls = big.logits(0), small.logits(0)
    assert _close(lb, ls, tol)
    assert big.comm_status() == 0
    if mode != "fp8" and (ls.topk(2).values[0] - ls.topk(2).values[1]) > 0.05 * ls.abs().max():
        assert tb == ts
    big.close()
    small.close()


def test_forward_rows_equals_step_by_step(tiny):
    """Speculative verify: M rows at once == M single steps (tokens and state)."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    prompt = [11, 12, 13, 14, 15]
    a = qh.QwenEngine(cfg, max_context=256, prefill_chunk=8).load(d)
    b = qh.QwenEngine(cfg, max_context=256, prefill_chunk=8).load(d)
    fa, fb = a.prefill(prompt), b.prefill(prompt)
    assert fa == fb
    seq = [fa] + a.decode(4)                       # plain greedy: 5 tokens
    rows = b.forward_rows(seq[:4])                 # feed the first 4 as a perfect draft
    assert rows == seq[1:5]                        # each row predicts its successor
    assert a.decode(3) == b.decode(3)              # same state afterwards
    a.close()
    b.close()


def test_random_init_runs_and_is_deterministic():
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    outs = []
    for _ in range(2):
        eng = qh.QwenEngine(cfg, max_context=128, prefill_chunk=32).init_random(seed=3, sigma=0.05)
        outs.append(eng.generate([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12], 8))
        eng.close()
    assert outs[0] == outs[1]
    assert all(0 <= t < cfg.vocab_size for t in outs[0])


def test_snapshot_restore_rewinds_recurrent_state(tiny):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    e = qh.QwenEngine(cfg, max_context=256, prefill_chunk=8).load(d)
    e.prefill([5, 6, 7, 8, 9, 10])
    snap = e.snapshot()
    first = e.decode(6)
    assert e.position == snap.position + 6
    snap.restore()
    assert e.position == snap.position and e.decode(6) == first
    snap.restore()
    e.forward_rows([1, 2, 3])                      # a rejected draft pollutes the state ...
    snap.restore()
    assert e.decode(6) == first                    # ... and the rewind removes it
    snap.free()
    e.close()


def test_speculative_decoding_equals_greedy(tiny):
    """Perfect, wrong and n-gram drafts all reproduce plain greedy decoding token for token."""
    from pocketllm_b200.models import qwen_hybrid as qh
    from pocketllm_b200.runtime.speculative import NGramDrafter, ReplayDrafter, speculative_generate
    cfg, tensors, d = tiny
    prompt = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    # plain steps and verify rows must round alike for token-for-token equality: both on the per-projection kernels
    e = qh.QwenEngine(cfg, max_context=256, prefill_chunk=8, persistent_decode=0).load(d)
    ref = e.generate(prompt, 33)
    n = len(prompt) + 1
    e.reset()
    out, st = speculative_generate(e, prompt, 33, ReplayDrafter(ref[1:], n), k=4)
    assert out == ref and st.acceptance == 1.0 and st.tokens_per_pass > 4.0
    e.reset()
    wrong = [(t + 1) % cfg.vocab_size for t in ref[1:]]
    out, st = speculative_generate(e, prompt, 33, ReplayDrafter(wrong, n), k=3)
    assert out == ref and st.accepted == 0
    e.reset()
    half = [t if i % 3 else (t + 7) % cfg.vocab_size for i, t in enumerate(ref[1:])]
    out, st = speculative_generate(e, prompt, 33, ReplayDrafter(half, n), k=7)
    assert out == ref and 0 < st.acceptance < 1
    e.reset()
    out, _ = speculative_generate(e, prompt, 33, NGramDrafter(), k=4)
    assert out == ref
    e.close()


def test_native_server_serves_the_engine(tiny):
    """pocket_engine --serve: the tokens behind the HTTP answer are the engine's greedy tokens."""
    import http.client
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path
    from pocketllm_b200.models import qwen_hybrid as qh
    from pocketllm_b200.server.cpp_sidecar import CharTokenizer
    cfg, tensors, d = tiny
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.Popen([str(root / "pocketllm_b200" / "_C" / "pocket_engine"), "--ckpt", str(d), "--serve", "--port", "0", "--tokenizer", "chars",
                             "--chat-format", "plain", "--sidecar-python", sys.executable, "--allow-shutdown", "--max-context", "512"],
                            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    try:
        line = proc.stdout.readline()
        assert line.startswith("openai_server_listening"), proc.stderr.read()
        port = int(dict(kv.split("=") for kv in line.split()[1:])["port"])
        body = {"messages": [{"role": "user", "content": "abc"}], "max_tokens": 12}
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
        c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
        out = json.loads(c.getresponse().read())
        c.close()
        prompt = CharTokenizer("plain").encode_chat(body["messages"])
        assert all(t < cfg.vocab_size for t in prompt)
        eng = qh.QwenEngine(cfg, max_context=512).load(d)
        want = eng.generate(prompt, 12)
        eng.close()
        if 0 in want:
            want = want[:want.index(0)]
        assert out["usage"]["prompt_tokens"] == len(prompt)
        assert out["choices"][0]["message"]["content"] == "".join(chr(t) for t in want)
        # a token outside the vocabulary is refused, and the server keeps serving
        c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
        c.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": "\uff5c"}], "max_tokens": 4}), {"Content-Type": "application/json"})
        r = c.getresponse()
        assert r.status == 400 and "vocabulary" in json.loads(r.read())["error"]["message"]
        c.close()
        # sampled request: different seeds give different continuations, the same seed repeats
        texts = []
        for seed in (1, 1, 2):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
            c.request("POST", "/v1/chat/completions", json.dumps(dict(body, temperature=1.5, seed=seed)), {"Content-Type": "application/json"})
            texts.append(json.loads(c.getresponse().read())["choices"][0]["message"]["content"])
            c.close()
        assert texts[0] == texts[1] and texts[0] != texts[2]
    finally:
        try:
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
            c.request("POST", "/shutdown", "{}")
            c.getresponse().read()
            proc.wait(timeout=30)
        except Exception:
            proc.kill()


def test_prefix_cache_reuses_state_across_requests(tiny):
    """A snapshot with KV rows taken at a block boundary survives an unrelated request in between."""
    from pocketllm_b200.models import qwen_hybrid as qh
    from pocketllm_b200.runtime.prefix_snapshot import PrefixSnapshotCache
    cfg, tensors, d = tiny
    e = qh.QwenEngine(cfg, max_context=256, prefill_chunk=8).load(d)
    cache = PrefixSnapshotCache(capacity=2, block=8, on_evict=lambda s: s.state.free())
    shared = [(7 * i + 3) % 1000 for i in range(19)]
    a, b = shared + [5, 6, 7], shared + [9, 8, 7, 6]
    other = [(11 * i + 1) % 1000 for i in range(40)]
    want_a, want_b = e.generate(a, 6), None
    e.reset()
    want_b = e.generate(b, 6)
    e.reset()
    got_a, reused_a = e.generate_cached(a, 6, cache)
    assert got_a == want_a and reused_a == 0 and cache.stats["captures"] == 1
    e.reset()
    e.generate(other, 4)                                   # overwrites KV rows and recurrent state
    got_b, reused_b = e.generate_cached(b, 6, cache)
    assert reused_b == 16 and got_b == want_b
    got_a2, reused_a2 = e.generate_cached(a, 6, cache)
    assert reused_a2 == 16 and got_a2 == want_a
    cache.clear()
    e.close()


@pytest.fixture(scope="module")
def tiny_mtp(tmp_path_factory):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4, hidden=256, inter=512, vocab=1024)
    out = {}
    for name, bf16_lin in (("fp8", False), ("bf16", True)):
        tensors = qh.random_checkpoint(cfg, seed=2, sigma=0.05, mtp=True, mtp_bf16_linears=bf16_lin)
        d = tmp_path_factory.mktemp("tiny_qwen_mtp_" + name)
        qh.save_checkpoint(d, cfg, tensors)
        out[name] = (tensors, d)
    return cfg, out


@pytest.mark.parametrize("variant,n_prompt", [("fp8", 6), ("fp8", 45), ("bf16", 21)])
def test_mtp_predictor_matches_oracle(tiny_mtp, variant, n_prompt):
    """After prefill the predictor has seen (hidden of position i, token i + 1) for the whole prompt plus the first
    generated token; its pick and logits agree with the fp32 definition, on the streaming and the tensor-core path."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, variants = tiny_mtp
    tensors, d = variants[variant]
    g = torch.Generator().manual_seed(n_prompt)
    prompt = torch.randint(0, cfg.vocab_size, (n_prompt,), generator=g).tolist()
    ref = qh.ReferenceModel(cfg, tensors)
    hid = []
    for t in prompt:
        logits = ref.step(t)
        hid.append(ref.last_hidden)
    eng = qh.QwenEngine(cfg, max_context=256, prefill_chunk=32, mtp=True).load(d)
    first = eng.prefill(prompt)
    if first != int(logits.argmax()):
        # only a near-tie of the target's logits may be decided differently; the predictor is then compared on the
        # engine's pick (its last row takes the token the target has just produced)
        top2 = logits.topk(2).values
        assert (top2[0] - top2[1]).item() < 0.02 * logits.abs().max().item()
        assert first == int(logits.topk(2).indices[1])
    shifted = prompt[1:] + [first]
    for i, (t, h) in enumerate(zip(shifted, hid)):
        mlogits, _ = ref.mtp_step(t, h, i)
    got = eng.mtp_logits()
    assert _close(got, mlogits, 5e-2)
    top2 = mlogits.topk(2).values
    if (top2[0] - top2[1]).item() > 0.05 * mlogits.abs().max().item():
        assert eng.mtp_next_token == int(mlogits.argmax())
    eng.close()


def test_mtp_speculative_decode_equals_plain_decode(tiny_mtp):
    """Same tokens as plain greedy decode, whatever the drafts are worth: with the predictor's own picks, with perfect
    drafts (every round accepted, draft length doubling), and with drafts that go wrong now and then (rewind + replay)."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, variants = tiny_mtp
    tensors, d = variants["fp8"]
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (53,), generator=g).tolist()
    n = 48
    eng = qh.QwenEngine(cfg, max_context=256, prefill_chunk=32, mtp=True).load(d)
    plain = eng.generate(prompt, n)
    eng.reset()
    spec, st = eng.generate_mtp(prompt, n, max_draft=4)
    assert spec == plain
    assert st["rounds"] >= 1 and st["proposed"] >= st["rounds"] and 0 <= st["accepted"] <= st["proposed"]
    assert st["accepted"] + st["rounds"] + st["plain_steps"] == n - 1
    # perfect drafts
    eng.reset()
    eng.set_draft_replay(plain[1:])
    spec, st = eng.generate_mtp(prompt, n, max_draft=4)
    assert spec == plain
    assert st["accepted"] == st["proposed"] and st["rollbacks"] == 0
    assert st["rounds"] <= 14 and st["proposed"] / st["rounds"] > 2.5          # 1, 2, 4, 4, ... drafts per round
    # drafts with an error every seventh token
    bad = [t if (i % 7) != 5 else (t + 1) % cfg.vocab_size for i, t in enumerate(plain[1:])]
    eng.reset()
    eng.set_draft_replay(bad)
    spec, st = eng.generate_mtp(prompt, n, max_draft=7)
    assert spec == plain
    assert st["rollbacks"] >= 3 and st["replay_tokens"] >= st["rollbacks"] and st["accepted"] < st["proposed"]
    # plain decode and speculative decode can alternate on one engine
    eng.set_draft_replay([])
    eng.reset()
    first = eng.prefill(prompt)
    a = eng.decode(5)
    b, _ = eng.spec_decode(10, 3)
    c = eng.decode(4)
    assert [first] + a + b + c == plain[:20]
    assert eng.comm_status() == 0
    eng.close()


def test_engine_without_predictor_rejects_spec_decode(tiny):
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    eng = qh.QwenEngine(cfg, max_context=128, prefill_chunk=32).load(d)
    eng.prefill([1, 2, 3])
    with pytest.raises(qh.EngineError):
        eng.spec_decode(4)
    eng.close()
    with pytest.raises(qh.EngineError):
        qh.QwenEngine(cfg, max_context=128, prefill_chunk=32, mtp=True).load(d)      # checkpoint has no mtp.* tensors


def test_native_server_with_multi_token_predictor(tiny_mtp):
    """pocket_engine --serve --qwen-mtp: greedy requests run through speculative decode in chunks and return the same text
    as plain greedy decoding; the speculative counters are printed when the server stops."""
    import http.client
    import json
    import os
    import subprocess
    import sys
    from pathlib import Path
    from pocketllm_b200.models import qwen_hybrid as qh
    from pocketllm_b200.server.cpp_sidecar import CharTokenizer
    cfg, variants = tiny_mtp
    tensors, d = variants["fp8"]
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.Popen([str(root / "pocketllm_b200" / "_C" / "pocket_engine"), "--ckpt", str(d), "--serve", "--port", "0", "--tokenizer", "chars",
                             "--chat-format", "plain", "--sidecar-python", sys.executable, "--allow-shutdown", "--max-context", "512",
                             "--qwen-mtp-tokens", "3"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    port = None
    try:
        line = proc.stdout.readline()
        assert line.startswith("openai_server_listening"), proc.stderr.read()
        port = int(dict(kv.split("=") for kv in line.split()[1:])["port"])
        eng = qh.QwenEngine(cfg, max_context=512).load(d)
        for content, n in (("hello there", 21), ("abc", 9)):
            body = {"messages": [{"role": "user", "content": content}], "max_tokens": n}
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
            c.request("POST", "/v1/chat/completions", json.dumps(body), {"Content-Type": "application/json"})
            out = json.loads(c.getresponse().read())
            c.close()
            eng.reset()
            want = eng.generate(CharTokenizer("plain").encode_chat(body["messages"]), n)
            if 0 in want:
                want = want[:want.index(0)]
            assert out["choices"][0]["message"]["content"] == "".join(chr(t) for t in want)
        eng.close()
    finally:
        try:
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=20)
            c.request("POST", "/shutdown", "{}")
            c.getresponse().read()
            rest = proc.communicate(timeout=30)[0]
        except Exception:
            proc.kill()
            rest = ""
    stats = dict(kv.split("=") for l in rest.splitlines() if l.startswith("serve_mtp_rounds") for kv in l.split())
    assert int(stats["serve_mtp_rounds"]) > 0 and int(stats["serve_mtp_proposed"]) >= int(stats["serve_mtp_accepted"])


def test_native_prefix_reuse_across_requests(tiny):
    """Sequential requests through the engine's own prefix reuse: a chat that grows (live continuation), a prompt that
    diverges in the middle (roll back to a stored recurrent state), an unrelated prompt (from zero). Tokens always
    equal those of a fresh engine."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    fresh = qh.QwenEngine(cfg, max_context=512, prefill_chunk=64, persistent_decode=0).load(d)
    eng = qh.QwenEngine(cfg, max_context=512, prefill_chunk=64, persistent_decode=0).load(d)
    eng.configure_prefix_cache(True, snapshot_interval=16, max_snapshots=6)
    fresh.configure_prefix_cache(True, snapshot_interval=16, max_snapshots=6)
    torch.manual_seed(11)
    base = torch.randint(0, cfg.vocab_size, (70,)).tolist()

    def want(prompt, n):
        # from zero, cut into the same pieces (a piece of other length takes other kernels and rounds differently)
        fresh.clear_prefix_cache()
        fresh.reset()
        first, st = fresh.prefill_reusing(prompt)
        assert st["reused_tokens"] == 0
        return [first] + fresh.decode(n - 1)

    def got(prompt, n):
        first, st = eng.prefill_reusing(prompt)
        return [first] + eng.decode(n - 1), st

    out1, st = got(base, 6)
    assert out1 == want(base, 6) and st["source"] == "empty" and st["reused_tokens"] == 0 and st["snapshots"] == 5   # 16, 32, 48, 64, 70
    # the conversation continues: old prompt + the reply + a new turn -> everything consumed so far is reused
    turn2 = base + out1[:5] + [7, 8, 9]
    out2, st = got(turn2, 5)
    assert out2 == want(turn2, 5)
    assert st["source"] == "live" and st["reused_tokens"] == 75 and st["computed_tokens"] == 3
    # a prompt that shares 40 tokens: the state stored at 32 serves, 32 tokens are not recomputed
    fork = base[:40] + [1, 2, 3, 4, 5, 6]
    out3, st = got(fork, 4)
    assert out3 == want(fork, 4)
    assert st["source"] == "snapshot" and st["reused_tokens"] == 32 and st["matched_tokens"] == 40
    # the same prompt once more: its own boundary state (46) is one token too far, the one at 32 serves again
    out4, st = got(fork, 4)
    assert out4 == out3 and st["source"] == "snapshot" and st["reused_tokens"] == 32
    # nothing in common
    other = [(t + 1) % cfg.vocab_size for t in base[:20]]
    out5, st = got(other, 4)
    assert out5 == want(other, 4) and st["source"] == "empty" and st["hits"] == 3 and st["misses"] == 2
    # switched off: reset + one prefill of the whole prompt
    eng.configure_prefix_cache(False)
    out6, st = got(other, 4)
    assert len(out6) == 4 and st["reused_tokens"] == 0 and st["source"] == "empty"
    assert eng.comm_status() == 0
    fresh.close()
    eng.close()


@pytest.mark.parametrize("persistent", [0, 1])
def test_fp8_kv_cache_tracks_the_bf16_cache(tiny, persistent):
    """The FP8 KV cache (E4M3 codes, one scale per 64 channels) changes the logits only slightly and takes a little over
    half the bytes; prefill, the per-projection decode and the persistent decode kernel all read and write it."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    torch.manual_seed(21)
    prompt = torch.randint(0, cfg.vocab_size, (90,)).tolist()
    outs = {}
    for dt in ("bf16", "fp8"):
        eng = qh.QwenEngine(cfg, max_context=512, prefill_chunk=64, persistent_decode=persistent, kv_cache_dtype=dt).load(d)
        first = eng.prefill(prompt)
        l0 = eng.logits(0)
        toks = [first] + eng.decode(6)
        outs[dt] = (toks, l0, eng.logits(0), eng.kv_cache_bytes)
        assert eng.persistent_decode == bool(persistent) and eng.comm_status() == 0
        eng.close()
    assert _close(outs["fp8"][1], outs["bf16"][1], 5e-2)          # after prefill
    if outs["fp8"][0] == outs["bf16"][0]:
        assert _close(outs["fp8"][2], outs["bf16"][2], 5e-2)      # after six decode steps on the same tokens
    assert outs["fp8"][0][0] == outs["bf16"][0][0]
    assert outs["fp8"][3] * 32 == outs["bf16"][3] * 17            # (128 + 2 * 4) bytes per row against 256


def test_canary_words_around_every_engine_buffer_stay_intact(tiny, monkeypatch):
    """POCKET_CANARY=1: guard bytes before and behind every device buffer; prefill (tensor-core and streaming paths),
    decode (persistent and per-projection) and verify rows leave all of them untouched."""
    from pocketllm_b200.models import qwen_hybrid as qh
    cfg, tensors, d = tiny
    monkeypatch.setenv("POCKET_CANARY", "1")
    torch.manual_seed(2)
    prompt = torch.randint(0, cfg.vocab_size, (150,)).tolist()
    for persistent in (1, 0):
        eng = qh.QwenEngine(cfg, max_context=512, prefill_chunk=64, persistent_decode=persistent).load(d)
        eng.prefill(prompt)
        toks = eng.decode(12)
        eng.forward_rows(toks[:5])
        eng.verify_canaries()
        eng.close()
    monkeypatch.delenv("POCKET_CANARY")
    plain = qh.QwenEngine(cfg, max_context=512, prefill_chunk=64).load(d)
    with pytest.raises(qh.EngineError, match="canaries are off"):
        plain.verify_canaries()
    plain.close()
