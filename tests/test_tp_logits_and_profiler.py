import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pocketllm_b200.moe.gate_profiler import GateProfiler
from pocketllm_b200.parallel import tp_logits


def test_vocab_row_range_covers_everything():
    for vocab, world in ((10, 3), (129280, 8), (7, 8)):
        spans = [tp_logits.vocab_row_range(vocab, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == vocab
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    vocab = 37
    full = torch.randn(5, vocab)
    full[0, 3] = full[0, 30] = 9.0                 # a tie across ranks: lowest id wins
    lo, hi = tp_logits.vocab_row_range(vocab, world, rank)
    ids = tp_logits.distributed_argmax(full[:, lo:hi], vocab)
    gathered = tp_logits.gather_logits(full[:, lo:hi], vocab)
    if rank == 0:
        q.put((ids.tolist(), torch.equal(gathered, full), full.argmax(-1).tolist()))
    dist.destroy_process_group()


def test_distributed_argmax_and_gather_three_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in ps:
        p.start()
    ids, same, ref = q.get(timeout=120)
    for p in ps:
        p.join(60)
    assert same and ids[0] == 3 and ids[1:] == ref[1:]


def test_gate_profiler_counts():
    gp = GateProfiler(8)
    gp.observe(0, torch.tensor([[0, 1], [2, 3]]))
    gp.predict(1, torch.tensor([[0, 5, 6], [3, 4, 7]]))
    gp.observe(1, torch.tensor([[0, 2], [3, 4]]))
    assert gp.hit_rate(1) == 0.75                       # 0, 3, 4 predicted; 2 missed
    s = gp.summary()
    assert s[1]["tokens_routed"] == 4 and s[1]["overlap_with_previous"] == 0.5
    assert gp.hot_experts(0) == [0, 1, 2, 3]
