"""A peer all-reduce that timed out on ONE rank must fail the step on EVERY rank and move all of them to the
library all-reduce together (CPU ranks over gloo; the peer object is a stand-in whose status word is set by hand)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


class _FakePeer:
    """Mimics the peer-memory all-reduce without any collective call: a healthy rank gets the sum (every rank r
    contributes r + 1 in this test), a rank whose status word is set keeps its local data, as the kernel does."""
    capacity = 1 << 20

    def __init__(self, world: int):
        self.total, self.word = float(sum(range(1, world + 1))), 0
        self.calls = 0

    def all_reduce(self, y):
        self.calls += 1
        if self.word == 0:
            y.fill_(self.total)
        return y

    def status(self, clear: bool = False) -> int:
        s = self.word
        if clear:
            self.word = 0
        return s


def _worker(rank, world, port, q):
    from pocketllm_b200.parallel.combine import ExpertCombine, StepFailed
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comb = ExpertCombine(world, None, peer=_FakePeer(world))
    y = torch.full((8,), float(rank + 1))
    comb(y)
    comb.check_step("cpu")                                   # clean step: nothing raised
    clean = y.tolist()
    comb.peer.word = 1 if rank == 1 else 0                   # rank 1's wait runs out during the next step
    y = torch.full((8,), float(rank + 1))
    comb(y)                                                  # rank 1 keeps its local partial sum: a wrong result
    raised = False
    try:
        comb.check_step("cpu")
    except StepFailed:
        raised = True
    y = torch.full((8,), float(rank + 1))
    comb(y)                                                  # every rank is on the library path now
    comb.check_step("cpu")
    q.put((rank, clean, raised, comb.peer is None, comb.calls["nccl"], y.tolist(), comb.fallbacks))
    dist.destroy_process_group()


def test_timeout_on_one_rank_fails_the_step_everywhere_and_switches_all_ranks():
    world = 3
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(world))
    for p in ps:
        p.join(60)
    total = float(sum(range(1, world + 1)))
    for rank, clean, raised, peer_off, nccl_calls, y, fallbacks in res:
        assert clean == [total] * 8
        assert raised, f"rank {rank} returned from a step another rank lost"
        assert peer_off and nccl_calls == 1 and fallbacks == 1
        assert y == [total] * 8


def test_single_rank_never_checks():
    from pocketllm_b200.parallel.combine import ExpertCombine
    c = ExpertCombine(1)
    y = torch.ones(4)
    assert c(y) is y
    c.check_step()


class _FakeMm(_FakePeer):
    def all_reduce(self, y, two_shot=None):
        self.shots = getattr(self, "shots", []) + [two_shot]
        return super().all_reduce(y)


def _worker_mm(rank, world, port, q):
    from pocketllm_b200.parallel.combine import ExpertCombine, StepFailed
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comb = ExpertCombine(world, None, peer=_FakePeer(world), mm=_FakeMm(world), multimem_min_floats=64)
    small, large = torch.full((8,), float(rank + 1)), torch.full((256,), float(rank + 1))
    comb(small)
    comb(large)
    comb.check_step("cpu")
    routed = (comb.calls["peer"], comb.calls["multimem"], comb.mm.shots)
    comb.mm.word = 1 if rank == 0 else 0                      # the in-switch path's wait runs out on rank 0
    raised = False
    try:
        comb.check_step("cpu")
    except StepFailed:
        raised = True
    y = torch.full((256,), float(rank + 1))
    comb(y)
    q.put((rank, routed, small.tolist()[0], large.tolist()[0], raised, comb.peer is None and comb.mm is None, comb.calls["nccl"], y.tolist()[0]))
    dist.destroy_process_group()


def test_large_payloads_take_the_in_switch_path_and_its_timeout_fails_the_step_everywhere():
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker_mm, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=180) for _ in range(world))
    for p in ps:
        p.join(60)
    for rank, routed, s0, l0, raised, all_off, nccl_calls, y0 in res:
        assert routed == (1, 1, [True])                       # 8 floats: unicast kernel; 256 floats: multimem, two shot
        assert s0 == l0 == 3.0
        assert raised and all_off and nccl_calls == 1 and y0 == 3.0
