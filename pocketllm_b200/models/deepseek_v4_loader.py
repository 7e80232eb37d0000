"""DeepSeek-V4 checkpoints on disk: Safetensors directory in the reference's tensor naming and
precision layout (reference: src/models/deepseek_v4/loader.py:440-675 `load_original_hf_model`;
Appendix-level facts: FP8 E4M3 weights with E8M0 scales per 128x128 block for the attention and
shared-expert linears, FP4 E2M1 + E8M0 per 32 for routed experts, bf16 for `wo_a`, compressor /
indexer projections, norms and embeddings, fp32 for the hyper-connection parameters).

`save_checkpoint` writes that layout from an fp32 weight dict (quantising the dense linears);
`load_checkpoint` returns (config, weights) with quantised tensors kept quantised:
`<name>.weight` float8_e4m3fn / uint8 nibbles and `<name>.scale` uint8 E8M0 codes.
"""
from __future__ import annotations

import json
import re
from pathlib import Path

import torch

from ..formats import fp8 as fp8fmt
from ..formats import safetensors_io as st
from . import deepseek_v4 as d4

_FP8_LINEAR = re.compile(r"\.(attn\.(wq_a|wq_b|wkv|wo_b)|shared_experts\.(w1|w2|w3)|e_proj|h_proj)\.weight$")
_BF16 = re.compile(r"(embed\.weight|head\.weight|norm\.weight|\.wo_a\.weight|compressor\.(wkv|wgate)\.weight|indexer\.(wq_b|weights_proj)\.weight|attn_sink)$")


def quantize_fp8_e8m0(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 [N, K] -> (E4M3 codes, E8M0 codes [ceil(N/128), ceil(K/128)]) with power-of-two block scales."""
    N, K = w.shape
    B = fp8fmt.BLOCK
    nb, kb = (N + B - 1) // B, (K + B - 1) // B
    wp = torch.zeros(nb * B, kb * B)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, B, kb, B)
    code = fp8fmt.float_to_e8m0(blocks.abs().amax(dim=(1, 3)).clamp_min(1e-30) / fp8fmt.E4M3_MAX)
    s = fp8fmt.e8m0_to_float(code).view(nb, 1, kb, 1)
    q = (blocks / s).clamp(-fp8fmt.E4M3_MAX, fp8fmt.E4M3_MAX).reshape(nb * B, kb * B)[:N, :K].contiguous()
    return q.to(torch.float8_e4m3fn), code


def dequantize_fp8_e8m0(q: torch.Tensor, code: torch.Tensor) -> torch.Tensor:
    return fp8fmt.dequantize_block128(q, fp8fmt.e8m0_to_float(code.view(torch.uint8)))


def save_checkpoint(directory: str | Path, cfg: d4.DSV4Config, W: dict[str, torch.Tensor], fp8_dense: bool = True) -> None:
    out: dict[str, torch.Tensor] = {}
    for name, t in W.items():
        if name.endswith(".scale") or t.dtype in (torch.uint8, torch.int32):
            out[name] = t
        elif fp8_dense and _FP8_LINEAR.search(name) and t.dim() == 2:
            q, code = quantize_fp8_e8m0(t)
            out[name], out[name[:-len("weight")] + "scale"] = q, code
        elif t.dtype == torch.bfloat16 or _BF16.search(name) or (t.dim() == 1 and "hc_" not in name):
            out[name] = t.to(torch.bfloat16)
        else:
            out[name] = t.float()
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(cfg.to_json())
    st.write_sharded(d, out, max_shard_bytes=1 << 30)


def load_checkpoint(directory: str | Path) -> tuple[d4.DSV4Config, dict[str, torch.Tensor]]:
    d = Path(directory)
    cfg = d4.DSV4Config.from_json((d / "config.json").read_text())
    model = st.SafetensorsModel(d)
    W = {}
    for k in model.keys():
        t = model.get(k)
        if k.endswith(".scale") and t.dtype != torch.uint8:
            t = t.view(torch.uint8)                   # E8M0 codes, whatever dtype tag the writer used
        W[k] = t
    return cfg, W


def dense_view(W: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """Copy of `W` with every FP8 linear dequantised to fp32 (for the oracle); FP4 experts stay packed."""
    out = {}
    for k, t in W.items():
        if t.dtype == torch.float8_e4m3fn:
            out[k] = dequantize_fp8_e8m0(t, W[k[:-len("weight")] + "scale"])
        elif k.endswith(".scale") and k[:-len("scale")] + "weight" in W and W[k[:-len("scale")] + "weight"].dtype == torch.float8_e4m3fn:
            continue
        else:
            out[k] = t.float() if t.is_floating_point() else t
    return out
