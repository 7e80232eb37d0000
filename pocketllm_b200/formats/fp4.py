"""FP4 E2M1 expert weights with one E8M0 scale per 32 values along the input dimension
(two codes per byte, low nibble first; value table {0, .5, 1, 1.5, 2, 3, 4, 6} with the sign
in bit 3). Reference: cpp_engine/cuda/fp4_ops.cu:34-70, src/kernels/ops.py:45-48."""
from __future__ import annotations

import torch

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
GROUP = 32


def quantize_e2m1(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 [..., K] -> (uint8 [..., K/2] packed codes, uint8 [..., K/32] E8M0 scales)."""
    *lead, K = w.shape
    if K % GROUP:
        raise ValueError(f"K={K} is not a multiple of {GROUP}")
    g = w.float().reshape(*lead, K // GROUP, GROUP)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -126)
    exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scale = torch.pow(2.0, exp)
    t = (g / scale[..., None]).clamp(-6.0, 6.0)
    idx = (t.abs()[..., None] - E2M1_VALUES).abs().argmin(-1)          # nearest magnitude
    code = idx.to(torch.uint8) | ((t < 0).to(torch.uint8) << 3)
    code = code.reshape(*lead, K)
    packed = code[..., 0::2] | (code[..., 1::2] << 4)
    return packed.contiguous(), (exp + 127).to(torch.uint8).contiguous()


def dequantize_e2m1(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    *lead, half = packed.shape
    K = half * 2
    lo, hi = packed & 15, packed >> 4
    code = torch.stack([lo, hi], dim=-1).reshape(*lead, K).long()
    val = E2M1_VALUES.to(code.device)[code & 7] * torch.where((code & 8) != 0, -1.0, 1.0)
    s = torch.pow(2.0, scales.float() - 127.0).repeat_interleave(GROUP, dim=-1)
    return val * s
