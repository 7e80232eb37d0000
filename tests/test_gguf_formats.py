"""GGUF container and block codecs (CPU): the dequantisers are checked against the
independent implementation in the `gguf` package, the quantisers by round trip."""
import numpy as np
import pytest

from pocketllm_b200.formats import gguf, gguf_quants as gq

gguf_py = pytest.importorskip("gguf")
from gguf import quants as oracle  # noqa: E402

ORACLE = {"q8_0": oracle.Q8_0, "q2_k": oracle.Q2_K, "q3_k": oracle.Q3_K, "q4_k": oracle.Q4_K, "q5_k": oracle.Q5_K,
          "q6_k": oracle.Q6_K, "iq2_xxs": oracle.IQ2_XXS, "iq2_xs": oracle.IQ2_XS, "iq3_xxs": oracle.IQ3_XXS,
          "iq4_xs": oracle.IQ4_XS, "iq1_m": oracle.IQ1_M}


def _random_blocks(name, n, seed=0):
    rng = np.random.default_rng(seed)
    _, qk, bs = gguf.GGML_TYPES[gguf.GGML_TYPE_IDS[name]]
    b = rng.integers(0, 256, size=(n, bs), dtype=np.uint8)
    # keep the fp16 scale fields finite and moderate
    def put_f16(col, lo=0.01, hi=0.1):
        b[:, col:col + 2] = rng.uniform(lo, hi, size=n).astype(np.float16)[:, None].view(np.uint8)
    if name == "q8_0":
        put_f16(0)
    elif name == "q2_k":
        put_f16(80), put_f16(82)
    elif name == "q3_k":
        put_f16(108)
    elif name in ("q4_k", "q5_k"):
        put_f16(0), put_f16(2)
    elif name == "q6_k":
        put_f16(208)
    elif name in ("iq2_xxs", "iq2_xs", "iq3_xxs", "iq4_xs"):
        put_f16(0)
    elif name == "iq1_m":
        # d is spread over the top nibbles of the four scale words: force a sane fp16
        d = rng.uniform(0.01, 0.1, size=n).astype(np.float16).view(np.uint16).astype(np.uint32)
        w = np.ascontiguousarray(b[:, 48:56]).view(np.uint16).astype(np.uint32) & 0x0FFF
        for i in range(4):
            w[:, i] |= ((d >> (4 * i)) & 0xF) << 12
        b[:, 48:56] = w.astype(np.uint16).view(np.uint8)
    return b


@pytest.mark.parametrize("name", sorted(ORACLE))
def test_dequantize_matches_gguf_package(name):
    b = _random_blocks(name, 64, seed=sum(map(ord, name)))
    mine = gq.dequantize(b[None], name)[0]
    if hasattr(ORACLE[name], "init_grid"):
        ORACLE[name].init_grid()               # the package fills its codebooks lazily
    ref = ORACLE[name].dequantize_blocks(b)
    assert mine.shape == ref.reshape(-1).shape or mine.reshape(ref.shape).shape == ref.shape
    np.testing.assert_allclose(mine.reshape(ref.shape), ref, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("name,tol", [("q8_0", 0.01), ("q5_k", 0.04), ("q4_k", 0.10), ("q2_k", 0.35),
                                      ("iq3_xxs", 0.25), ("iq2_xs", 0.40), ("iq2_xxs", 0.45), ("iq1_m", 0.65)])
def test_quantize_roundtrip(name, tol):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((6, 512)) * 0.02).astype(np.float32)
    blocks = gq.quantize(x, name)
    _, qk, bs = gguf.GGML_TYPES[gguf.GGML_TYPE_IDS[name]]
    assert blocks.shape == (6, 512 // qk, bs) and blocks.dtype == np.uint8
    back = gq.dequantize(blocks, name)
    rel = np.linalg.norm(back - x) / np.linalg.norm(x)
    assert rel < tol, rel
    # our blocks are valid for an independent decoder too
    ref = ORACLE[name].dequantize_blocks(blocks.reshape(-1, bs)).reshape(x.shape)
    np.testing.assert_allclose(back, ref, rtol=1e-5, atol=1e-7)


def test_quantize_zero_rows_are_finite():
    for name in gq.QUANTIZABLE:
        back = gq.dequantize(gq.quantize(np.zeros((2, 256), np.float32), name), name)
        assert np.isfinite(back).all() and np.abs(back).max() < 1e-3


def test_gguf_writer_reader_roundtrip(tmp_path):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    wr = gguf.GGUFWriter()
    wr.add_meta("general.architecture", "minimax-m2")
    wr.add_meta("minimax-m2.block_count", 2)
    wr.add_meta("minimax-m2.rope.freq_base", 5e6)
    wr.add_meta("tokenizer.ggml.tokens", ["a", "b", "c"])
    wr.add_meta("tokenizer.ggml.token_type", [1, 1, 3])
    wr.add_meta("flag", True)
    wr.add_tensor("blk.0.attn_q.weight", gq.quantize(w, "q5_k"), "q5_k", w.shape)
    wr.add_tensor("blk.0.ffn_gate_exps.weight", gq.quantize(np.stack([w, w * 2]), "iq2_xxs"), "iq2_xxs", (2, 8, 512))
    wr.add_tensor("output_norm.weight", np.ones(512, np.float32), "f32")
    p = tmp_path / "m.gguf"
    wr.write(p)
    f = gguf.GGUFFile(p)
    assert f.architecture() == "minimax-m2" and f.metadata["minimax-m2.block_count"] == 2
    assert f.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"] and f.metadata["flag"] is True
    assert abs(f.metadata["minimax-m2.rope.freq_base"] - 5e6) < 1
    t = f.tensors["blk.0.ffn_gate_exps.weight"]
    assert t.shape == (2, 8, 512) and t.type_name == "iq2_xxs" and t.nbytes == 2 * 8 * 2 * 66
    assert f.data_offset % 32 == 0 and all(ti.offset % 32 == 0 for ti in f.tensors.values())
    back = gq.dequantize(f.blocks("blk.0.attn_q.weight"), "q5_k")
    assert np.linalg.norm(back - w) / np.linalg.norm(w) < 0.04
    assert np.array_equal(gq.dequantize(f.raw("output_norm.weight"), "f32"), np.ones(512, np.float32))


def test_gguf_bundle_shards(tmp_path):
    for i in (1, 2):
        wr = gguf.GGUFWriter()
        wr.add_meta("general.architecture", "glm-dsa")
        wr.add_tensor(f"t{i}", np.full(32, i, np.float32), "f32")
        wr.write(tmp_path / f"model-{i:05d}-of-00002.gguf")
    b = gguf.GGUFBundle(tmp_path / "model-00001-of-00002.gguf")
    assert sorted(b.tensors) == ["t1", "t2"] and b.architecture() == "glm-dsa"
    assert gq.dequantize(b.raw("t2"), "f32")[0] == 2.0
    with pytest.raises(FileNotFoundError):
        (tmp_path / "model-00002-of-00002.gguf").unlink()
        gguf.GGUFBundle(tmp_path / "model-00001-of-00002.gguf")


def test_truncated_file_is_rejected(tmp_path):
    wr = gguf.GGUFWriter()
    wr.add_tensor("w", np.zeros(1024, np.float32), "f32")
    p = tmp_path / "t.gguf"
    wr.write(p)
    data = p.read_bytes()
    p.write_bytes(data[: len(data) - 100])
    with pytest.raises(ValueError):
        gguf.GGUFFile(p)
