import json

import pytest

from pocketllm_b200.config import Config
from pocketllm_b200.utils import trace


def test_config_precedence(tmp_path):
    f = tmp_path / "c.json"
    f.write_text(json.dumps({"model": {"path": "/m", "max_context": 8192}, "cache": {"prefill_chunk": 512}}))
    env = {"POCKET_CACHE_PREFILL_CHUNK": "128", "POCKET_PARALLEL_PEER_ALLREDUCE": "false", "UNRELATED": "x"}
    c = Config.load(f, profile="latency2", env=env, overrides=["serving.port=9001", "speculative.draft_len=3"])
    assert c.model.path == "/m" and c.model.max_context == 8192
    assert c.cache.prefill_chunk == 128                      # env beats file beats profile
    assert c.parallel.peer_allreduce is False and c.serving.port == 9001
    assert c.speculative.mode == "ngram" and c.speculative.draft_len == 3 and c.serving.max_queue == 2
    assert json.loads(c.dump())["serving"]["port"] == 9001


def test_config_rejects_bad_input(tmp_path):
    with pytest.raises(ValueError, match="unknown serving profile"):
        Config.load(profile="turbo", env={})
    with pytest.raises(ValueError, match="unknown config field"):
        Config.load(env={}, overrides=["cache.nope=1"])
    with pytest.raises(ValueError, match="not a boolean"):
        Config.load(env={"POCKET_CACHE_CUDA_GRAPH": "maybe"})
    with pytest.raises(ValueError, match="between 1 and 8"):
        Config.load(env={}, overrides=["parallel.world=16"])
    with pytest.raises(ValueError, match="layer_pp"):
        Config.load(env={}, overrides=["parallel.policy=layer_pp", "speculative.mode=mtp"])
    y = tmp_path / "c.yaml"
    y.write_text("parallel:\n  world: 4\nmodel:\n  family: deepseek_v4\n")
    assert Config.load(y, env={}).parallel.world == 4


def test_roofline_arithmetic():
    peaks = {"hbm_gbs": 6000.0, "bf16_tflops": 1500.0, "source": "measured"}
    r = trace.roofline(hbm_bytes=24e9, seconds=8e-3, peaks=peaks)
    assert r["limiter"] == "hbm" and abs(r["bound_s"] - 4e-3) < 1e-9 and abs(r["fraction_of_measured"] - 0.5) < 1e-9
    r = trace.roofline(flops=3e12, hbm_bytes=1e9, nvlink_bytes=7.7e9, seconds=0.02, peaks=peaks)
    assert r["limiter"] == "nvlink" and abs(r["bound_s"] - 0.01) < 1e-9
    r = trace.roofline(flops=3e15, hbm_bytes=1e9, seconds=4.0, peaks=peaks)
    assert r["limiter"] == "compute" and abs(r["achieved_tflops"] - 750.0) < 1e-6
    assert trace.measured_peaks()["hbm_gbs"] > 1000
    t = trace.SectionTimer(enabled=False, nvtx=False)
    with t.section("x"):
        pass
    assert t.summary() == {}


def test_device_memory_floor_decision():
    """POCKET_MIN_FREE_MIB: the engine refuses allocations that would leave less than the floor free (pure decision
    function of the native library, so no GPU is needed)."""
    import ctypes
    from pocketllm_b200.ops import lib
    if not lib.available("engine"):
        import pytest
        pytest.skip("libpocket_engine.so not built")
    L = lib.engine()
    buf = ctypes.create_string_buffer(400)
    MiB = 1 << 20
    fn = L.pk_mem_headroom_verdict
    fn.argtypes = [ctypes.c_ulonglong] * 4 + [ctypes.c_char_p, ctypes.c_int]
    assert fn(10000 * MiB, 180000 * MiB, 2000 * MiB, 4096 * MiB, buf, 400) == 0 and buf.value == b""
    assert fn(10000 * MiB, 180000 * MiB, 7000 * MiB, 4096 * MiB, buf, 400) == 1
    assert b"POCKET_MIN_FREE_MIB" in buf.value and b"7000.0 MiB" in buf.value and b"3000.0 MiB" in buf.value
    assert fn(1000 * MiB, 180000 * MiB, 7000 * MiB, 1 * MiB, buf, 400) == 1          # larger than what is free
    assert fn(1000 * MiB, 180000 * MiB, 7000 * MiB, 0, buf, 400) == 0                # no floor configured: cudaMalloc decides


def test_config_to_native_engine_flags():
    from pocketllm_b200.config import Config
    import pytest
    cfg = Config.load(overrides=["model.path=/ckpt/qwen", "model.max_context=8192", "parallel.world=2", "speculative.mode=mtp",
                                 "speculative.draft_len=3", "serving.native=true", "serving.port=9000", "model.tokenizer=/tok/dir",
                                 "model.chat_format=qwen", "cache.cuda_graph=false"])
    a = cfg.native_engine_args(rank=1)
    assert a[:2] == ["--ckpt", "/ckpt/qwen"] and a[a.index("--tp-rank") + 1] == "1" and a[a.index("--tp-world") + 1] == "2"
    assert "--no-cuda-graph" in a and a[a.index("--qwen-mtp-tokens") + 1] == "3"
    assert a[a.index("--tokenizer") + 1] == "hf:/tok/dir" and a[a.index("--port") + 1] == "9000" and "--serve" in a
    plain = Config.load(overrides=["model.path=/m"]).native_engine_args()
    assert "--serve" not in plain and "--qwen-mtp-tokens" not in plain
    with pytest.raises(ValueError):
        Config.load(overrides=["speculative.mode=ngram"]).native_engine_args()
    with pytest.raises(ValueError):
        Config.load(overrides=["speculative.mode=dspark", "model.family=qwen_hybrid"])
    Config.load(overrides=["speculative.mode=dspark", "model.family=deepseek_v4"])
