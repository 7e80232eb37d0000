"""Native DeepSeek-V4 config parser and the container-agnostic tensor lookup, against the Python writers."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from pocketllm_b200.models import deepseek_v4 as d4
from pocketllm_b200.models import deepseek_v4_gguf as dg
from pocketllm_b200.models import deepseek_v4_loader as ld

ROOT = Path(__file__).resolve().parent.parent
ENGINE = ROOT / "pocketllm_b200" / "_C" / "pocket_engine"


def _run(*args, ok=True):
    r = subprocess.run([str(ENGINE), *map(str, args)], capture_output=True, text=True, timeout=120)
    assert (r.returncode == 0) == ok, r.stdout + r.stderr
    return r.stdout + r.stderr


def _fields(line):
    out = {}
    for part in line.split():
        k, _, v = part.partition("=")
        out[k] = v
    return out


@pytest.fixture(scope="module")
def saved(tmp_path_factory):
    if not ENGINE.exists():
        pytest.skip("native engine binary not built")
    cfg = d4.DSV4Config.tiny()
    W = d4.random_checkpoint(cfg, seed=0)
    d = tmp_path_factory.mktemp("dsv4_ws")
    ld.save_checkpoint(d / "ck", cfg, W)
    dg.write_gguf(d / "m.gguf", cfg, W, dense_type="q8_0", expert_type="q4_k")
    return cfg, W, d / "ck", d / "m.gguf"


def test_dsv4_config_from_json_and_gguf(saved):
    cfg, W, ck, gg = saved
    want = json.loads(cfg.to_json())
    for src in (ck, gg):
        got = json.loads(_run("--dsv4-config", src).strip().splitlines()[-1])
        for k, v in want.items():
            assert got[k] == pytest.approx(v) if isinstance(v, float) else got[k] == v, k
    # tensor-parallel degrees that do not divide heads, output groups and experts are refused
    assert "must divide" in _run("--dsv4-config", ck, "--tp-world", "3", ok=False)
    _run("--dsv4-config", ck, "--tp-world", "2")


def test_dsv4_config_defaults_of_a_published_gguf(tmp_path):
    """A file that carries only the counts gets the V4-Flash shape for the rest, like the Python reader."""
    if not ENGINE.exists():
        pytest.skip("native engine binary not built")
    from pocketllm_b200.formats import gguf
    w = gguf.GGUFWriter()
    for k, v in {"general.architecture": "deepseek4", "deepseek4.block_count": 43, "deepseek4.expert_count": 256,
                 "deepseek4.expert_used_count": 6, "deepseek4.embedding_length": 4096}.items():
        w.add_meta(k, v)
    w.add_tensor("dummy", np.zeros(32, np.float32), "f32")
    w.write(tmp_path / "p.gguf")
    got = json.loads(_run("--dsv4-config", tmp_path / "p.gguf").strip().splitlines()[-1])
    ref = dg.config_from_metadata({"general.architecture": "deepseek4", "deepseek4.block_count": 43})
    assert got["n_layers"] == 43 and got["head_dim"] == ref.head_dim and got["n_mtp_layers"] == 0
    assert got["compress_ratios"] == list(ref.compress_ratios[:43])


def test_weight_source_lookup_in_both_containers(saved):
    cfg, W, ck, gg = saved
    # Safetensors: the model's names are the stored names
    f = _fields(_run("--weight-source", ck, "--lookup", "layers.1.attn.wq_a.weight").splitlines()[-1])
    assert f["found"] == "1" and f["stored"] == "layers.1.attn.wq_a.weight" and f["shape"] == f"[{cfg.q_lora_rank},{cfg.dim}]"
    # GGUF: translated names, GGUF dimension order reversed back to rows x columns
    out = _run("--weight-source", gg, "--lookup", "layers.1.attn.wq_a.weight").splitlines()
    assert out[0] == "format=gguf"
    f = _fields(out[-1])
    assert f["found"] == "1" and f["stored"] == "blk.1.attn_q_a.weight" and f["dtype"] == "q8_0"
    assert f["shape"] == f"[{cfg.q_lora_rank},{cfg.dim}]" and int(f["bytes"]) == cfg.q_lora_rank * cfg.dim // 32 * 34
    f = _fields(_run("--weight-source", gg, "--lookup", "hc_head_fn").splitlines()[-1])
    assert f["stored"] == "output_hc_fn.weight" and f["dtype"] == "f32"
    assert _fields(_run("--weight-source", gg, "--lookup", "layers.0.no.such.tensor").splitlines()[-1])["found"] == "0"
    # every name the GGUF source lists resolves
    listed = [l for l in _run("--weight-source", gg).splitlines() if l.startswith("tensor=")]
    assert len(listed) == len([n for n, _, _ in dg.tensor_plan(cfg) if "_exps" not in n]) and all("found=1" in l for l in listed)


def test_weight_source_expert_slices(saved):
    cfg, W, ck, gg = saved
    from pocketllm_b200.formats import gguf
    b = gguf.GGUFBundle(gg)
    E, I, d = cfg.n_routed_experts, cfg.moe_inter_dim, cfg.dim
    for part, name, rows, cols in (("w1", "ffn_gate_exps", I, d), ("w2", "ffn_down_exps", d, I), ("w3", "ffn_up_exps", I, d)):
        raw = np.asarray(b.raw(f"blk.2.{name}.weight")).reshape(E, -1)
        for e in (0, E - 1):
            f = _fields(_run("--weight-source", gg, "--lookup-expert", f"2,{e},{part}").splitlines()[-1])
            assert f["found"] == "1" and f["shape"] == f"[{rows},{cols}]" and f["dtype"] == "q4_k"
            assert int(f["bytes"]) == raw.shape[1] and int(f["byte_sum"]) == int(raw[e].astype(np.uint64).sum())
    # Safetensors keeps one tensor per expert
    f = _fields(_run("--weight-source", ck, "--lookup-expert", "2,3,w2").splitlines()[-1])
    assert f["found"] == "1" and f["stored"] == "layers.2.ffn.experts.3.w2.weight"
    assert "out of range" in _run("--weight-source", gg, "--lookup-expert", f"2,{E},w1", ok=False)
    assert "w1, w2 or w3" in _run("--weight-source", gg, "--lookup-expert", "2,0,w9", ok=False)
