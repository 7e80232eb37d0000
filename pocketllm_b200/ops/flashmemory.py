"""Long-context chunk scorer ("FlashMemory") bindings (`csrc/kernels/flashmemory.cu`): build the scorer query of one decode
token, score every compressed-KV chunk of a layer on the FP8 tensor cores, combine layers, pick the chunks to keep.

Reference counterpart: cpp_engine/include/flashmemory_ops.hpp (score_layer, score_layer_floatk, ensemble, topk,
write_global_indices, yarn_inv_freqs) and docs/FLASHMEMORY_1M_CONTEXT.md.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong
from dataclasses import dataclass

import torch

from . import _check, _ptr, _sm_count, _stream
from . import lib as _lib
from . import dsv4_ops as _dk

HEAD_DIM = 128


def yarn_inv_freqs(rope_dim: int, base: float, factor: float, original_seq_len: int, beta_fast: float, beta_slow: float) -> torch.Tensor:
    """[rope_dim / 2] angular frequency of every rotated pair: plain `base ** (-2i / rope_dim)` below the beta_fast
    correction dim, divided by `factor` above the beta_slow one, blended linearly in between."""
    freqs = 1.0 / (base ** (torch.arange(0, rope_dim, 2, dtype=torch.float64) / rope_dim))
    if original_seq_len > 0 and factor != 1.0:
        def corr(rot: float) -> float:
            return rope_dim * math.log(original_seq_len / (rot * 2 * math.pi)) / (2 * math.log(base))
        low, high = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), rope_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(rope_dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        freqs = freqs * (1 - ramp) + freqs / factor * ramp
    return freqs.float()


@dataclass
class ScorerWeights:
    """One scorer layer, fp32 on the device: wq_a [rank, hidden], wq_b [heads * 128, rank], q_norm [rank],
    weights_proj [heads, hidden], inv_freqs [rope_dim / 2]."""
    wq_a: torch.Tensor
    wq_b: torch.Tensor
    q_norm: torch.Tensor
    weights_proj: torch.Tensor
    inv_freqs: torch.Tensor
    eps: float = 1e-6

    @property
    def n_heads(self) -> int:
        return self.weights_proj.shape[0]

    @property
    def rope_dim(self) -> int:
        return 2 * self.inv_freqs.numel()


def quantize_keys(keys: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 chunk keys [n, 128] -> (E4M3 codes uint8 [n, 128], scale fp32 [n] = amax / 448)."""
    n = keys.shape[0]
    codes = torch.empty(n, HEAD_DIM, device=keys.device, dtype=torch.uint8)
    scale = torch.empty(n, device=keys.device, dtype=torch.float32)
    _check(_lib.kernels().pk_flashmemory_quant_keys(_ptr(keys.contiguous()), c_int(n), _ptr(codes), _ptr(scale), _stream()), "pk_flashmemory_quant_keys")
    return codes, scale


def unpack_keys(packed: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Rows of 128 code bytes followed by the 4 bytes of their fp32 scale (uint8 [n, 132]) -> (codes [n, 128], scale [n])."""
    n = packed.shape[0]
    codes = torch.empty(n, HEAD_DIM, device=packed.device, dtype=torch.uint8)
    scale = torch.empty(n, device=packed.device, dtype=torch.float32)
    _check(_lib.kernels().pk_flashmemory_unpack_keys(_ptr(packed.contiguous()), c_int(n), _ptr(codes), _ptr(scale), _stream()), "pk_flashmemory_unpack_keys")
    return codes, scale


def build_query(w: ScorerWeights, hidden: torch.Tensor, position: int, want_q: bool = False):
    """Scorer query of one token: (qcodes uint8 [256, 128], head_w fp32 [128][, q fp32 [heads, 128]])."""
    dev = hidden.device
    rank, hidden_dim = w.wq_a.shape
    qlora = torch.empty(rank, device=dev, dtype=torch.float32)
    qcodes = torch.empty(256, HEAD_DIM, device=dev, dtype=torch.uint8)
    head_w = torch.empty(128, device=dev, dtype=torch.float32)
    q = torch.empty(w.n_heads, HEAD_DIM, device=dev, dtype=torch.float32) if want_q else None
    st = _lib.kernels().pk_flashmemory_build_query(_ptr(hidden), _ptr(w.wq_a), _ptr(w.wq_b), _ptr(w.q_norm), _ptr(w.weights_proj), _ptr(w.inv_freqs),
                                                   c_int(w.n_heads), c_int(rank), c_int(hidden_dim), c_int(w.rope_dim), c_float(w.eps),
                                                   c_longlong(position), _ptr(qlora), _ptr(qcodes), _ptr(head_w), _ptr(q), _stream())
    _check(st, "pk_flashmemory_build_query")
    return (qcodes, head_w, q) if want_q else (qcodes, head_w)


def score_chunks(key_codes: torch.Tensor, key_scale: torch.Tensor, qcodes: torch.Tensor, head_w: torch.Tensor, *, sigmoid: bool = True,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """score[c] = f(sum_h relu(q[h] . k[c]) * w[h]) for every chunk, as one FP8 tensor-core GEMM over the keys."""
    n = key_codes.shape[0]
    dev = key_codes.device
    partial = torch.empty(4, n, device=dev, dtype=torch.float32)
    ones2 = torch.ones(2, device=dev, dtype=torch.float32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    scores = torch.empty(n, device=dev, dtype=torch.float32) if out is None else out
    st = _lib.kernels().pk_flashmemory_score_chunks(_ptr(key_codes), _ptr(key_scale), c_int(n), _ptr(qcodes), _ptr(head_w), _ptr(ones2), _ptr(partial),
                                                    c_int(int(sigmoid)), _ptr(scores), _ptr(status), c_int(_sm_count()), _stream())
    _check(st, "pk_flashmemory_score_chunks")
    return scores


def score_layer(w: ScorerWeights, hidden: torch.Tensor, key_codes: torch.Tensor, key_scale: torch.Tensor, position: int, sigmoid: bool = True) -> torch.Tensor:
    qcodes, head_w = build_query(w, hidden, position)
    return score_chunks(key_codes, key_scale, qcodes, head_w, sigmoid=sigmoid)


def ensemble(layer_scores: torch.Tensor, n_chunks: int, use_max: bool = True) -> torch.Tensor:
    """layer_scores fp32 [layers, stride >= n_chunks] -> max (or mean) over layers [n_chunks]."""
    out = torch.empty(n_chunks, device=layer_scores.device, dtype=torch.float32)
    st = _lib.kernels().pk_flashmemory_ensemble(_ptr(layer_scores), c_int(layer_scores.shape[0]), c_int(n_chunks), c_int(layer_scores.stride(0)),
                                                c_int(int(use_max)), _ptr(out), _stream())
    _check(st, "pk_flashmemory_ensemble")
    return out


def topk(scores: torch.Tensor, keep: int) -> tuple[torch.Tensor, torch.Tensor]:
    """The `keep` best chunks: (logical indices int32, their scores), best first. Selection is a device radix select;
    only the kept entries are sorted."""
    sel = _dk.topk_select(scores.view(1, -1), keep)[0]
    sel = sel[sel >= 0]
    vals = scores[sel.long()]
    order = torch.argsort(vals, descending=True, stable=True)
    return sel[order].contiguous(), vals[order].contiguous()


def write_global_indices(logical: torch.Tensor, offset: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Physical KV rows of logical chunks: `offset + id` (offset = the layer's window rows); -1 stays -1."""
    out = torch.empty_like(logical) if out is None else out
    st = _lib.kernels().pk_flashmemory_write_global_indices(_ptr(logical), c_int(logical.numel()), c_int(offset), _ptr(out), _stream())
    _check(st, "pk_flashmemory_write_global_indices")
    return out


# ---- fp32 definition (the oracle of the tests) ----

def _hadamard(n: int) -> torch.Tensor:
    h = torch.ones(1, 1)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def reference_query(w: ScorerWeights, hidden: torch.Tensor, position: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(q fp32 [heads, 128], head weights [heads]) by the definition, on the tensors' device."""
    ql = w.wq_a.float() @ hidden.float()
    ql = ql * torch.rsqrt(ql.square().mean() + w.eps) * w.q_norm.float()
    q = (w.wq_b.float() @ ql).view(w.n_heads, HEAD_DIM).to(torch.bfloat16).float()
    rd = w.rope_dim
    ang = position * w.inv_freqs.float()
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = q[:, HEAD_DIM - rd::2].clone(), q[:, HEAD_DIM - rd + 1::2].clone()
    q[:, HEAD_DIM - rd::2] = (a * c - b * s).to(torch.bfloat16).float()
    q[:, HEAD_DIM - rd + 1::2] = (a * s + b * c).to(torch.bfloat16).float()
    q = q @ _hadamard(HEAD_DIM).to(q.device) / math.sqrt(HEAD_DIM)
    hw = (w.weights_proj.float() @ hidden.float()) / math.sqrt(HEAD_DIM * w.n_heads)
    return q, hw


def reference_scores(w: ScorerWeights, hidden: torch.Tensor, keys: torch.Tensor, position: int, sigmoid: bool = True) -> torch.Tensor:
    q, hw = reference_query(w, hidden, position)
    x = (torch.relu(keys.float() @ q.t()) * hw).sum(-1)
    return torch.sigmoid(x) if sigmoid else x
