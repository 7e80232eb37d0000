"""Writes a random-init checkpoint of the Qwen3.8-27B-FP8 benchmark shape in the on-disk
format the reference engine loads (config.json + Safetensors shards with its tensor names:
FP8 E4M3 `weight` + BF16 `weight_scale_inv` per 128x128 block, BF16 norms / embeddings).

Weights are N(0, 0.02) values quantised to FP8 block by block; to keep the 27 GB write
fast, each matrix is assembled from a pool of quantised 128x128 blocks drawn at random.

    python -m baseline.make_qwen_checkpoint --out /dev/shm/qwen27b_random [--layers 64]
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from pocketllm_b200.formats import fp8 as fp8fmt  # noqa: E402
from pocketllm_b200.formats import safetensors_io as st_io  # noqa: E402
from pocketllm_b200.models.qwen_hybrid import QwenHybridConfig  # noqa: E402

POOL = 512  # quantised 128x128 blocks in the pool


def _pool(seed: int, sigma: float) -> tuple[np.ndarray, np.ndarray]:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(POOL * 128, 128, generator=g) * sigma
    q, s = fp8fmt.quantize_block128(w)
    return q.view(torch.uint8).numpy().reshape(POOL, 128, 128), s.view(torch.int16).numpy().reshape(POOL)


def _fp8_matrix(rng: np.random.Generator, pool_q: np.ndarray, pool_s: np.ndarray, n: int, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    nb, kb = n // 128, k // 128
    idx = rng.integers(0, POOL, size=(nb, kb))
    w = pool_q[idx].transpose(0, 2, 1, 3).reshape(n, k)          # [nb, 128, kb, 128] -> [n, k]
    s = pool_s[idx]
    return torch.from_numpy(np.ascontiguousarray(w)).view(torch.float8_e4m3fn), torch.from_numpy(np.ascontiguousarray(s)).view(torch.bfloat16)


def write_checkpoint(out: Path, cfg: QwenHybridConfig, seed: int = 0, sigma: float = 0.02) -> int:
    out.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(seed)
    pool_q, pool_s = _pool(seed, sigma)
    g = torch.Generator().manual_seed(seed + 1)
    H, D = cfg.hidden_size, cfg.head_dim
    prefix = "model.language_model."
    weight_map: dict[str, str] = {}
    total = 0

    def bf16(*shape, mean=0.0, std=sigma):
        return (mean + std * torch.randn(*shape, generator=g)).to(torch.bfloat16)

    def flush(name: str, tensors: dict[str, torch.Tensor]) -> None:
        nonlocal total
        st_io.write_file(out / name, tensors)
        for k, t in tensors.items():
            weight_map[k] = name
            total += t.numel() * t.element_size()

    def fp8(tensors, name, n, k):
        w, s = _fp8_matrix(rng, pool_q, pool_s, n, k)
        tensors[name + ".weight"] = w
        tensors[name + ".weight_scale_inv"] = s

    head = {prefix + "embed_tokens.weight": bf16(cfg.vocab_size, H), prefix + "norm.weight": bf16(H, std=0.05),
            "lm_head.weight": bf16(cfg.vocab_size, H)}
    flush("model-globals.safetensors", head)
    KD = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    VD = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    for i, kind in enumerate(cfg.layer_types):
        p = f"{prefix}layers.{i}."
        t: dict[str, torch.Tensor] = {p + "input_layernorm.weight": bf16(H, std=0.05), p + "post_attention_layernorm.weight": bf16(H, std=0.05)}
        if kind == "linear_attention":
            fp8(t, p + "linear_attn.in_proj_qkv", 2 * KD + VD, H)
            fp8(t, p + "linear_attn.in_proj_z", VD, H)
            fp8(t, p + "linear_attn.out_proj", H, VD)
            t[p + "linear_attn.in_proj_a.weight"] = bf16(cfg.linear_num_value_heads, H)
            t[p + "linear_attn.in_proj_b.weight"] = bf16(cfg.linear_num_value_heads, H)
            t[p + "linear_attn.conv1d.weight"] = bf16(2 * KD + VD, 1, cfg.linear_conv_kernel_dim, std=0.3)
            t[p + "linear_attn.A_log"] = bf16(cfg.linear_num_value_heads, std=0.5)
            t[p + "linear_attn.dt_bias"] = bf16(cfg.linear_num_value_heads, std=0.5)
            t[p + "linear_attn.norm.weight"] = bf16(cfg.linear_value_head_dim, mean=1.0, std=0.05)
        else:
            fp8(t, p + "self_attn.q_proj", cfg.num_attention_heads * D * 2, H)
            fp8(t, p + "self_attn.k_proj", cfg.num_key_value_heads * D, H)
            fp8(t, p + "self_attn.v_proj", cfg.num_key_value_heads * D, H)
            fp8(t, p + "self_attn.o_proj", H, cfg.num_attention_heads * D)
            t[p + "self_attn.q_norm.weight"] = bf16(D, std=0.05)
            t[p + "self_attn.k_norm.weight"] = bf16(D, std=0.05)
        fp8(t, p + "mlp.gate_proj", cfg.intermediate_size, H)
        fp8(t, p + "mlp.up_proj", cfg.intermediate_size, H)
        fp8(t, p + "mlp.down_proj", H, cfg.intermediate_size)
        flush(f"model-layer-{i:03d}.safetensors", t)
    (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}))
    d = json.loads(cfg.to_json())
    d["architectures"] = ["Qwen3_5ForCausalLM"]
    d["tie_word_embeddings"] = False
    (out / "config.json").write_text(json.dumps({"architectures": d["architectures"], "model_type": "qwen3_5", "text_config": d}))
    (out / ".complete").write_text(str(total))
    return total


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--tiny", action="store_true")
    args = ap.parse_args()
    cfg = QwenHybridConfig.tiny() if args.tiny else QwenHybridConfig.benchmark_27b()
    if args.layers != cfg.num_hidden_layers and not args.tiny:
        cfg.num_hidden_layers = args.layers
        cfg.layer_types = []
        cfg.__post_init__()
    n = write_checkpoint(Path(args.out), cfg)
    print(f"wrote {n / 1e9:.2f} GB to {args.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
