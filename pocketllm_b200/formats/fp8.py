"""FP8 E4M3 block-scaled weights (the Safetensors layout of Qwen-FP8 and DeepSeek FP8
checkpoints): `weight` holds E4M3 codes, `weight_scale_inv[ceil(N/128), ceil(K/128)]` the
multiplier of each 128x128 block, so that `w = e4m3(code) * scale_inv[n // 128, k // 128]`
(reference: cpp_engine/cuda/qwen_half_ops.cu:89-113, cpp_engine/src/qwen_weights.cpp:618-655).
"""
from __future__ import annotations

import torch

BLOCK = 128
E4M3_MAX = 448.0


def quantize_block128(w: torch.Tensor, scale_dtype: torch.dtype = torch.bfloat16) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 [N, K] -> (float8_e4m3fn [N, K], scale_inv [ceil(N/128), ceil(K/128)])."""
    N, K = w.shape
    nb, kb = (N + BLOCK - 1) // BLOCK, (K + BLOCK - 1) // BLOCK
    wp = torch.zeros(nb * BLOCK, kb * BLOCK, dtype=torch.float32)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, BLOCK, kb, BLOCK)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = (amax / E4M3_MAX).to(scale_dtype)          # stored precision
    q = blocks / scale.float().view(nb, 1, kb, 1)
    q = q.clamp(-E4M3_MAX, E4M3_MAX).reshape(nb * BLOCK, kb * BLOCK)[:N, :K].contiguous()
    return q.to(torch.float8_e4m3fn), scale


def dequantize_block128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Inverse of `quantize_block128`, fp32."""
    N, K = q.shape
    s = scale.float().repeat_interleave(BLOCK, 0)[:N].repeat_interleave(BLOCK, 1)[:, :K]
    return q.float() * s


def e8m0_to_float(code: torch.Tensor) -> torch.Tensor:
    """E8M0 exponent-only scale: 2 ** (code - 127)."""
    return torch.pow(2.0, code.to(torch.float32) - 127.0)


def float_to_e8m0(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x, as an E8M0 code (uint8)."""
    e = torch.ceil(torch.log2(x.clamp_min(2.0 ** -127)))
    return (e + 127).clamp(0, 254).to(torch.uint8)
