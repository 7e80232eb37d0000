"""Serving engine: batching of compatible whole-completion requests, and the rank-0 / worker protocol of the Python
server under several ranks (CPU ranks over gloo, a counting stand-in for the model)."""
import os
import socket
import threading
import time

import torch.distributed as dist
import torch.multiprocessing as mp

from pocketllm_b200.server.engine import SamplingParams, ServingEngine, batch_compatible


class _EchoBatchBackend:
    """Token i of a completion is prompt[0] + i; records how requests were grouped."""
    max_batch_size = 4

    def __init__(self):
        self.calls = []

    def generate(self, prompt_ids, p):
        self.calls.append(("single", 1))
        for i in range(p.max_tokens):
            yield prompt_ids[0] + i

    def generate_batch(self, prompts, params):
        self.calls.append(("batch", len(prompts)))
        time.sleep(0.01)
        return [[pr[0] + i for i in range(p.max_tokens)] for pr, p in zip(prompts, params)]


def _collect(engine, prompt, params, batchable, out, key):
    out[key] = [t for t in engine.stream(prompt, params, batchable=batchable) if not isinstance(t, tuple)]


def test_compatible_completions_share_a_batch_and_streams_run_alone():
    be = _EchoBatchBackend()
    eng = ServingEngine(be, batch_wait_ms=200.0)
    out, threads = {}, []
    for k in range(3):
        threads.append(threading.Thread(target=_collect, args=(eng, [100 * (k + 1)], SamplingParams(max_tokens=3 + k), True, out, k)))
    for t in threads:
        t.start()
    for t in threads:
        t.join(20)
    assert out == {0: [100, 101, 102], 1: [200, 201, 202, 203], 2: [300, 301, 302, 303, 304]}
    assert ("batch", 3) in be.calls or (("batch", 2) in be.calls)          # the window caught at least two of them
    assert eng.stats["batched_requests"] >= 2 and eng.stats["requests"] == 3
    # a stream never joins a batch; another sampler setting does not either
    be.calls.clear()
    _collect(eng, [7], SamplingParams(max_tokens=2), False, out, "s")
    assert out["s"] == [7, 8] and be.calls == [("single", 1)]
    assert batch_compatible(SamplingParams(max_tokens=5), SamplingParams(max_tokens=9))
    assert not batch_compatible(SamplingParams(temperature=0.7, seed=1), SamplingParams(temperature=0.7, seed=2))
    assert not batch_compatible(SamplingParams(), SamplingParams(top_k=5))
    eng.close()


def test_incompatible_request_found_while_batching_still_runs():
    be = _EchoBatchBackend()
    eng = ServingEngine(be, batch_wait_ms=300.0)
    out = {}
    a = threading.Thread(target=_collect, args=(eng, [10], SamplingParams(max_tokens=2), True, out, "a"))
    b = threading.Thread(target=_collect, args=(eng, [20], SamplingParams(max_tokens=2, top_k=3, temperature=0.5, seed=1), True, out, "b"))
    a.start()
    time.sleep(0.05)
    b.start()
    a.join(20)
    b.join(20)
    assert out["a"] == [10, 11] and out["b"] == [20, 21]
    eng.close()


class _CountingBackend:
    def __init__(self):
        self.seen = []

    def generate(self, prompt_ids, p):
        self.seen.append((list(prompt_ids), p.max_tokens, p.stop_token_ids))
        for i in range(p.max_tokens):
            tok = prompt_ids[-1] + i + 1
            yield tok
            if tok in p.stop_token_ids:
                return


def _rank(rank, world, port, q):
    from pocketllm_b200.server import distributed
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    group = distributed.control_group()
    be = _CountingBackend()
    if rank == 0:
        front = distributed.DistributedBackend(be, group)
        full = list(front.generate([1, 2, 3], SamplingParams(max_tokens=4)))
        it = front.generate([5], SamplingParams(max_tokens=6, stop_token_ids=(9,)))
        early = [next(it), next(it)]
        it.close()                                           # the client went away after two tokens
        front.shutdown()
        q.put((rank, full, early, be.seen))
    else:
        served = distributed.worker_loop(be, group)
        q.put((rank, served, None, be.seen))
    dist.destroy_process_group()


def test_workers_follow_rank_zero_and_finish_abandoned_requests():
    world = 3
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(world))
    for p in ps:
        p.join(60)
    (_, full, early, seen0), (_, served1, _, seen1), (_, served2, _, seen2) = res
    assert full == [4, 5, 6, 7] and early == [6, 7]
    assert served1 == served2 == 2
    assert seen0 == seen1 == seen2 == [([1, 2, 3], 4, ()), ([5], 6, (9,))]
