"""CPU routed-experts backend (worker thread), the shared-memory expert server process and the weight arena."""
import os
import subprocess
import sys
import uuid
from pathlib import Path

import pytest
import torch

from pocketllm_b200.moe import cpu_oracle as co
from pocketllm_b200.moe import ipc, moe_server
from pocketllm_b200.moe.cpu_backend import CPURoutedExpertsBackend

ROOT = Path(__file__).resolve().parent.parent


def _layers():
    return {0: co.random_fp4_moe(256, 128, 4, shared=True, seed=1), 3: co.random_fp4_moe(256, 128, 4, shared=False, seed=2)}


def test_backend_submit_sync_matches_reference():
    layers = _layers()
    be = CPURoutedExpertsBackend(layers, topk=2)
    x = torch.randn(5, 256)
    be.submit(0, x)
    with pytest.raises(RuntimeError, match="in flight"):
        be.submit(3, x)
    y = be.sync()
    ref, _ = co.forward_torch(x, layers[0], topk=2)
    assert torch.allclose(y, ref, atol=2e-4, rtol=1e-3)
    assert torch.allclose(be.forward(3, x), co.forward_torch(x, layers[3], topk=2)[0], atol=2e-4, rtol=1e-3)
    with pytest.raises(RuntimeError, match="without submit"):
        be.sync()
    with pytest.raises(KeyError):
        be.submit(7, x)
    assert be.stats["calls"] == 2 and be.stats["tokens"] == 10
    be.close()


def test_weight_arena_roundtrip_and_timeout():
    name = "pk_arena_" + uuid.uuid4().hex[:8]
    layers = _layers()
    arena = ipc.SharedWeightArena.create(name, moe_server.pack_layers(layers))
    other = ipc.SharedWeightArena.attach(name, timeout_s=5)
    got = moe_server.unpack_layers(other)
    assert torch.equal(got[0].w13, layers[0].w13) and torch.equal(got[3].router, layers[3].router) and got[3].shared_w13 is None
    del got
    other.close()
    arena.close()
    with pytest.raises(TimeoutError):
        ipc.SharedWeightArena.attach("pk_arena_missing_" + uuid.uuid4().hex[:6], timeout_s=0.2)


def test_server_process_serves_and_stops():
    tag = uuid.uuid4().hex[:8]
    layers = _layers()
    arena = ipc.SharedWeightArena.create("pk_a_" + tag, moe_server.pack_layers(layers))
    chans = [ipc.MoEChannel(f"pk_c{i}_{tag}", 16, 256, create=True) for i in range(2)]
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.Popen([sys.executable, "-m", "pocketllm_b200.moe.moe_server", "--arena", "pk_a_" + tag, "--channels",
                             ",".join(c.name for c in chans), "--max-tokens", "16", "--hidden", "256", "--topk", "2"], env=env)
    try:
        for c in chans:
            c.wait_until_ready(120)
        x = torch.randn(7, 256)
        for layer in (0, 3, 0):
            for c in chans:
                y = c.request(layer, x, timeout_s=60)
                assert torch.allclose(y, co.forward_torch(x, layers[layer], topk=2)[0], atol=2e-4, rtol=1e-3)
        with pytest.raises(ValueError):
            chans[0].request(0, torch.randn(17, 256))
        proc.terminate()                                   # SIGTERM: the server flags STOP on its way out
        proc.wait(timeout=30)
        with pytest.raises(ipc.ServerStopped):
            chans[0].request(0, x, timeout_s=5)
    finally:
        if proc.poll() is None:
            proc.kill()
        for c in chans:
            c.close()
        arena.close()


def test_client_times_out_when_nobody_serves():
    c = ipc.MoEChannel("pk_lonely_" + uuid.uuid4().hex[:8], 4, 64, create=True)
    try:
        with pytest.raises(TimeoutError, match="did not become ready"):
            c.wait_until_ready(0.1)
        with pytest.raises(TimeoutError, match="did not answer"):
            c.request(0, torch.zeros(2, 64), timeout_s=0.2)
    finally:
        c.close()


def test_backend_runs_int8_experts():
    """The asynchronous CPU backend takes INT8 experts (per-row scales) as well as FP4 ones."""
    import torch
    from pocketllm_b200.moe import cpu_oracle as co
    from pocketllm_b200.moe.cpu_backend import CPURoutedExpertsBackend
    from pocketllm_b200.ops import lib
    import pytest
    if not lib.available("cpu"):
        pytest.skip("libpocket_cpu.so not built")
    g = torch.Generator().manual_seed(2)
    E, I, H, k, T = 6, 64, 96, 2, 5
    router = torch.randn(E, H, generator=g) * 0.05
    w13, w2 = torch.randn(E, 2 * I, H, generator=g) * 0.05, torch.randn(E, H, I, generator=g) * 0.05
    w = co.Int8MoEWeights.quantize(router, w13, w2)
    assert w.dims == (E, I, H) and w.w13.dtype == torch.int8
    be = CPURoutedExpertsBackend({3: w}, k, score_func="sigmoid", norm_topk=True)
    x = torch.randn(T, H, generator=g)
    y = be.forward(3, x)
    be.close()
    # fp32 math on the dequantised weights
    d13, d2 = w.w13.float() * w.s13.unsqueeze(-1), w.w2.float() * w.s2.unsqueeze(-1)
    sc = torch.sigmoid(x @ router.T)
    top = sc.topk(k, -1)
    wt = top.values / top.values.sum(-1, keepdim=True)
    ref = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(top.indices[t, j])
            gu = d13[e] @ x[t]
            ref[t] += wt[t, j] * (d2[e] @ (torch.nn.functional.silu(gu[:I]) * gu[I:]))
    assert torch.allclose(y, ref, atol=1e-4, rtol=1e-3)
    assert int(be.last_counts.sum()) == T * k
