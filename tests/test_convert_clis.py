"""Checkpoint converters on tiny synthetic inputs (CPU)."""
import numpy as np
import torch

from pocketllm_b200.cli import convert_checkpoint, make_routed_source_gguf
from pocketllm_b200.formats import fp4, gguf, gguf_quants
from pocketllm_b200.models import deepseek_v4 as d4
from pocketllm_b200.models import deepseek_v4_loader as ld


def test_convert_checkpoint_directions(tmp_path):
    cfg = d4.DSV4Config.tiny(n_layers=1, n_mtp_layers=0, compress_ratios=(4, 0), n_routed_experts=2, n_hash_layers=0)
    W = d4.random_checkpoint(cfg, seed=3)
    ld.save_checkpoint(tmp_path / "fp8", cfg, W)
    assert convert_checkpoint.main(["--hf-ckpt-path", str(tmp_path / "fp8"), "--save-path", str(tmp_path / "bf16"), "--dense", "bf16", "--experts", "bf16"]) == 0
    _, A = ld.load_checkpoint(tmp_path / "fp8")
    _, B = ld.load_checkpoint(tmp_path / "bf16")
    assert B["layers.0.attn.wq_b.weight"].dtype == torch.bfloat16 and "layers.0.attn.wq_b.scale" not in B
    assert torch.equal(B["layers.0.attn.wq_b.weight"].float(), ld.dense_view(A)["layers.0.attn.wq_b.weight"])      # exact dequantisation
    e = "layers.0.ffn.experts.1.w2"
    assert torch.equal(B[e + ".weight"].float(), fp4.dequantize_e2m1(A[e + ".weight"], A[e + ".scale"]))
    # and back: quantising the dequantised checkpoint reproduces the codes (values are exactly representable)
    assert convert_checkpoint.main(["--hf-ckpt-path", str(tmp_path / "bf16"), "--save-path", str(tmp_path / "again"), "--dense", "fp8", "--experts", "mxfp4"]) == 0
    _, C = ld.load_checkpoint(tmp_path / "again")
    assert torch.equal(ld.dense_view(C)["layers.0.attn.wq_b.weight"], ld.dense_view(A)["layers.0.attn.wq_b.weight"])
    assert torch.equal(fp4.dequantize_e2m1(C[e + ".weight"], C[e + ".scale"]), fp4.dequantize_e2m1(A[e + ".weight"], A[e + ".scale"]))


def test_make_routed_source_gguf(tmp_path):
    cfg = d4.DSV4Config.tiny(n_layers=2, n_mtp_layers=0, compress_ratios=(0, 0, 0), n_routed_experts=3, n_hash_layers=0)
    W = d4.random_checkpoint(cfg, seed=4)
    ld.save_checkpoint(tmp_path / "hf", cfg, W)
    E, I, H = 3, cfg.moe_inter_dim, cfg.dim
    tpl = gguf.GGUFWriter()
    tpl.add_meta("general.architecture", "deepseek4")
    tpl.add_meta("tokenizer.ggml.tokens", ["a", "b", "c"])
    tpl.add_tensor("token_embd.weight", np.ones((4, H), np.float32), "f32")
    for l in range(2):
        for part, shape in (("gate", (E, I, H)), ("up", (E, I, H)), ("down", (E, H, I))):
            tpl.add_tensor(f"blk.{l}.ffn_{part}_exps.weight", gguf_quants.quantize(np.zeros((E * shape[1], shape[2]), np.float32), "q8_0").reshape(E, shape[1], -1, 34), "q8_0", shape)
    tpl.write(tmp_path / "tpl.gguf")
    out = tmp_path / "out.gguf"
    assert make_routed_source_gguf.main(["--template-gguf", str(tmp_path / "tpl.gguf"), "--hf-ckpt-path", str(tmp_path / "hf"), "--output", str(out),
                                         "--dry-run"]) == 0 and not out.exists()
    assert make_routed_source_gguf.main(["--template-gguf", str(tmp_path / "tpl.gguf"), "--hf-ckpt-path", str(tmp_path / "hf"), "--output", str(out),
                                         "--layers", "1", "--target-type", "f16"]) == 0
    f = gguf.GGUFFile(out)
    assert f.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"] and f.tensors["blk.0.ffn_up_exps.weight"].type_name == "q8_0"
    t = f.tensors["blk.1.ffn_down_exps.weight"]
    assert t.type_name == "f16" and tuple(t.shape) == (E, H, I)
    got = np.frombuffer(f.raw("blk.1.ffn_down_exps.weight"), dtype=np.float16).reshape(E, H, I)
    want = fp4.dequantize_e2m1(W["layers.1.ffn.experts.2.w2.weight"], W["layers.1.ffn.experts.2.w2.scale"]).numpy()
    np.testing.assert_array_equal(got[2].astype(np.float32), want.astype(np.float16).astype(np.float32))
    assert make_routed_source_gguf.main(["--template-gguf", str(tmp_path / "tpl.gguf"), "--hf-ckpt-path", str(tmp_path / "hf"), "--output", str(out)]) == 2
