"""Safetensors writer/reader and FP8 block-128 quantisation round trips (CPU)."""
import json

import torch

from pocketllm_b200.formats import fp8, safetensors_io as st


def test_fp8_block_roundtrip():
    torch.manual_seed(0)
    w = torch.randn(300, 260) * 0.02
    q, s = fp8.quantize_block128(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (3, 3)
    back = fp8.dequantize_block128(q, s)
    rel = (back - w).abs().max() / w.abs().max()
    assert rel < 0.07  # 3 mantissa bits
    # quantising the dequantised tensor again is exact (codes are stable)
    q2, s2 = fp8.quantize_block128(back)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) or (fp8.dequantize_block128(q2, s2) - back).abs().max() < 1e-3


def test_e8m0_codes():
    x = torch.tensor([1.0, 0.5, 3.0, 2.0 ** -10])
    c = fp8.float_to_e8m0(x)
    assert c.tolist() == [127, 126, 129, 117]
    assert torch.allclose(fp8.e8m0_to_float(c), torch.tensor([1.0, 0.5, 4.0, 2.0 ** -10]))


def test_safetensors_file_roundtrip(tmp_path):
    t = {
        "a.weight": torch.randn(4, 8).to(torch.bfloat16),
        "b": torch.arange(12, dtype=torch.int32).view(3, 4),
        "c.weight": (torch.randn(128, 128) * 0.02).to(torch.float8_e4m3fn),
        "empty": torch.zeros(0, dtype=torch.float32),
    }
    p = tmp_path / "x.safetensors"
    st.write_file(p, t, {"format": "pt"})
    f = st.SafetensorsFile(p)
    assert f.metadata == {"format": "pt"}
    for k, v in t.items():
        got = f.get(k)
        assert got.dtype == v.dtype and list(got.shape) == list(v.shape)
        assert torch.equal(got.view(torch.uint8), v.view(torch.uint8))


def test_safetensors_sharded(tmp_path):
    t = {f"layer.{i}.w": torch.randn(64, 64) for i in range(6)}
    files = st.write_sharded(tmp_path, t, max_shard_bytes=40000)
    assert len(files) == 3
    idx = json.loads((tmp_path / "model.safetensors.index.json").read_text())
    assert set(idx["weight_map"]) == set(t)
    m = st.SafetensorsModel(tmp_path)
    for k, v in t.items():
        assert torch.equal(m.get(k), v)
