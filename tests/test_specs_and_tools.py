"""Specs, capability / placement reports, inspect CLI, imatrix, prewarm on synthetic GGUFs (CPU)."""
import json

import numpy as np
import pytest

from pocketllm_b200.cli import inspect_gguf, merge_imatrix
from pocketllm_b200.formats import gguf, imatrix, prewarm
from pocketllm_b200.models import glm_dsa, minimax_m2
from pocketllm_b200.moe import spec


@pytest.fixture(scope="module")
def files(tmp_path_factory):
    d = tmp_path_factory.mktemp("gg")
    minimax_m2.write_random_gguf(d / "mm.gguf", minimax_m2.MiniMaxM2Config.tiny())
    glm_dsa.write_random_gguf(d / "glm.gguf", glm_dsa.GLMDSAConfig.tiny())
    return d


def test_spec_params_validation_capability(files):
    b = gguf.GGUFBundle(files / "mm.gguf")
    p = spec.parse_params(b)
    assert p.architecture == "minimax-m2" and p.n_routed_experts == 8 and p.top_k == 2 and p.hidden_size == 256
    assert spec.validate(b).ok
    c = spec.capability(b)
    assert c.supported and set(c.per_type_bytes) == {"f32", "q4_k", "q5_k", "iq2_xxs"}
    g = gguf.GGUFBundle(files / "glm.gguf")
    assert spec.parse_params(g).leading_dense_layers == 1 and spec.validate(g).ok


def test_validation_reports_missing_and_wrong_shape(files, tmp_path):
    src = gguf.GGUFFile(files / "mm.gguf")
    w = gguf.GGUFWriter()
    for k, v in src.metadata.items():
        if k != "general.alignment":
            w.add_meta(k, v, src.metadata_types[k])
    for name, t in src.tensors.items():
        if name == "blk.1.attn_q.weight":
            continue
        if name == "output_norm.weight":
            w.add_tensor(name, np.ones(128, np.float32), "f32")
        else:
            w.add_tensor(name, src.raw(name), t.type_name, t.shape)
    w.write(tmp_path / "bad.gguf")
    v = spec.validate(gguf.GGUFBundle(tmp_path / "bad.gguf"))
    assert not v.ok and v.missing == ["blk.1.attn_q.weight"] and any("output_norm" in s for s in v.wrong_shape)


def test_placement_modes(files):
    b = gguf.GGUFBundle(files / "mm.gguf")
    assert spec.placement(b).mode == "resident"
    tiny_hw = spec.HardwareProfile(n_gpus=2, hbm_gib=1e-3, reserve_fraction=0.0)   # ~1 MiB per GPU
    r = spec.placement(b, tiny_hw)
    assert r.mode in ("host_staged", "does_not_fit")


def test_inspect_cli(files, capsys):
    rc = inspect_gguf.main([str(files / "glm.gguf"), "--summary", "--spec-summary", "--validate-spec", "--capability-report",
                            "--placement-report", "--json"])
    out = json.loads(capsys.readouterr().out)
    assert rc == 0 and out["summary"]["tensors"] > 20 and out["validation"]["ok"] and out["placement"]["mode"] == "resident"


def test_imatrix_collect_merge(tmp_path):
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((10, 64)).astype(np.float32), rng.standard_normal((6, 64)).astype(np.float32)
    c1, c2 = imatrix.IMatrixCollector(), imatrix.IMatrixCollector()
    c1.observe("blk.0.ffn_down.weight", a)
    c2.observe("blk.0.ffn_down.weight", b)
    c1.save(tmp_path / "a.gguf")
    c2.save(tmp_path / "b.gguf")
    assert merge_imatrix.main([str(tmp_path / "m.gguf"), str(tmp_path / "a.gguf"), str(tmp_path / "b.gguf")]) == 0
    m = imatrix.load(tmp_path / "m.gguf")
    assert m.counts["blk.0.ffn_down.weight"] == 16
    np.testing.assert_allclose(imatrix.importance(m, "blk.0.ffn_down.weight"), (np.concatenate([a, b]) ** 2).mean(0), rtol=1e-5)


def test_prewarm_reads_all_bytes(files):
    r = prewarm.prewarm(files / "mm.gguf", chunk_mib=1)
    assert r["bytes"] == (files / "mm.gguf").stat().st_size and r["files"] == 1


def test_minimax_rope_table_lookup_equals_direct_rotation():
    """The device-table rotation used by the MiniMax runtime gives the values of the direct (fp64 angle) rotation."""
    import torch
    from pocketllm_b200.models.minimax_m2 import _rope, _rope_lookup, _rope_tables
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 3, 128, generator=g)
    pos = torch.tensor([0, 1, 5, 17, 63, 64, 99], dtype=torch.int32)
    cos_t, sin_t = _rope_tables(128, 64, 5.0e6, "cpu")
    assert cos_t.shape == (128, 32) and cos_t.dtype == torch.float32
    assert torch.equal(_rope_lookup(x, pos, cos_t, sin_t, 64), _rope(x, pos, 64, 5.0e6))
    assert torch.equal(_rope_lookup(x, pos, cos_t, sin_t, 64)[..., 64:], x[..., 64:])      # dims past rope_dim pass through


def test_validate_ds4_q2_checks_metadata_and_expert_block_types(tmp_path, capsys):
    """A minimal deepseek4 file with the published 2-bit layout passes; a wrong expert type, a missing tensor and a
    missing metadata key are each named."""
    import json
    import numpy as np
    from pocketllm_b200.formats import gguf

    def write(path, down_type="q2_k", drop=None, skip_meta=None):
        w = gguf.GGUFWriter()
        w.add_meta("general.architecture", "deepseek4")
        for k, v in (("deepseek4.block_count", 2), ("deepseek4.embedding_length", 256), ("deepseek4.expert_count", 2),
                     ("deepseek4.expert_used_count", 1), ("deepseek4.expert_feed_forward_length", 256)):
            if k != skip_meta:
                w.add_meta(k, v)
        for layer in range(2):
            for suffix, typ in inspect_gguf.DS4_Q2_EXPERT_TYPES:
                name = f"blk.{layer}.{suffix}"
                if name == drop:
                    continue
                typ = down_type if suffix == "ffn_down_exps.weight" else typ
                shape = (2, 256, 256) if "_exps" in suffix else (256, 256)
                nbytes = gguf.tensor_nbytes(gguf.GGML_TYPE_IDS[typ], shape)
                w.add_tensor(name, np.zeros(nbytes, dtype=np.uint8), typ, shape)
        w.write(path)

    write(tmp_path / "ok.gguf")
    assert inspect_gguf.main([str(tmp_path / "ok.gguf"), "--validate-ds4-q2", "--json"]) == 0
    assert json.loads(capsys.readouterr().out)["ds4_q2_validation"] == {"ok": True, "problems": [], "more": 0}
    write(tmp_path / "bad.gguf", down_type="q4_k", drop="blk.1.ffn_up_shexp.weight", skip_meta="deepseek4.expert_count")
    assert inspect_gguf.main([str(tmp_path / "bad.gguf"), "--validate-ds4-q2", "--json"]) == 1
    problems = json.loads(capsys.readouterr().out)["ds4_q2_validation"]["problems"]
    assert "missing metadata deepseek4.expert_count" in problems
    assert "missing tensor blk.1.ffn_up_shexp.weight" in problems
    assert "blk.0.ffn_down_exps.weight is q4_k, expected q2_k" in problems and len(problems) == 4
