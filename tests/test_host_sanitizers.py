"""The engine's host C++ (JSON, readers, sampler, rendezvous, command channel, protocol model) built with
AddressSanitizer + UndefinedBehaviorSanitizer, and the protocol model again under ThreadSanitizer."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SRC = [ROOT / "csrc" / "tests" / "host_selftest.cpp"] + [ROOT / "csrc" / "engine" / f for f in
                                                        ("json.cpp", "gguf_reader.cpp", "safetensors.cpp", "sampler.cpp", "control_plane.cpp")]
GXX = shutil.which("g++", path="/usr/bin") or shutil.which("g++")


def _inputs(tmp_path):
    from pocketllm_b200.models import minimax_m2, qwen_hybrid as qh
    minimax_m2.write_random_gguf(tmp_path / "m.gguf", minimax_m2.MiniMaxM2Config.tiny())
    cfg = qh.QwenHybridConfig.tiny(layers=2, hidden=128, inter=256, vocab=256)
    qh.save_checkpoint(tmp_path / "st", cfg, qh.random_checkpoint(cfg, seed=0))
    (tmp_path / "scratch").mkdir()
    return [str(tmp_path / "m.gguf"), str(tmp_path / "st"), str(tmp_path / "scratch")]


@pytest.mark.skipif(GXX is None, reason="no g++")
@pytest.mark.parametrize("flags", ["-fsanitize=address,undefined -fno-sanitize-recover=all", "-fsanitize=thread"])
def test_host_selftest_under_sanitizers(tmp_path, flags):
    exe = tmp_path / "host_selftest"
    cmd = [GXX, "-std=c++17", "-O1", "-g", "-pthread", *flags.split(), *map(str, SRC), "-o", str(exe)]
    b = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if b.returncode != 0 and ("cannot find -l" in b.stderr or "libasan" in b.stderr or "libtsan" in b.stderr or "libubsan" in b.stderr):
        pytest.skip("sanitizer runtime is not installed")
    assert b.returncode == 0, b.stderr[-3000:]
    r = subprocess.run([str(exe), *_inputs(tmp_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "host_selftest=ok" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
