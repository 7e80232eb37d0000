"""GLM-5-class "glm-dsa" on raw GGUF blocks: MLA attention with a DSA lightning indexer,
leading dense SwiGLU layers, then routed MoE (sigmoid scores, bias for selection, optional
normalisation, expert_weights_scale) plus one shared expert.

Numerical contract (reference: src/models/glm_dsa/architecture.py:263-877):
  q = q_b(rmsnorm(q_a(x))) -> [H, key_mla_dim]; kv_a_mqa(x) -> [kv_lora_rank | rope_dim];
  latent = rmsnorm(kv_lora part); k_nope = latent k_b, v = latent v_b; the rope part of k is
  shared by all heads; q's last rope_dim dims rotate; RoPE pairs are interleaved (2i, 2i+1);
  softmax scale 1/sqrt(key_mla_dim).
The reference validates the indexer tensors but never runs them (spec.py:94-126). Here the
indexer is implemented (score_t,c = sum_h w_h relu(q_h . k_c), top-k positions per query,
following the DSV4 indexer maths, src/models/deepseek_v4/runtime.py:1112-1288) and can be
switched off (`dsa_topk=0`) to compare with dense attention.

Tensor layout notes for this implementation: `attn_k_b.weight` is [heads, k_nope, kv_lora],
`attn_v_b.weight` is [heads, value_mla, kv_lora]; both are decoded to fp32 at load (they
are small). Every other matrix stays in raw blocks.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

import numpy as np
import torch

from ..formats import gguf, gguf_quants as gq

ARCH = "glm-dsa"


@dataclass
class GLMDSAConfig:
    vocab_size: int = 154880
    dim: int = 6144
    n_layers: int = 78
    leading_dense_layers: int = 3
    n_heads: int = 64
    q_lora_rank: int = 2048
    kv_lora_rank: int = 512
    key_mla_dim: int = 256        # nope + rope
    value_mla_dim: int = 256
    rope_dim: int = 64
    rope_theta: float = 1.0e6
    indexer_heads: int = 32
    indexer_key_dim: int = 128
    dsa_topk: int = 2048
    dense_inter: int = 12288
    n_experts: int = 256
    top_k: int = 8
    expert_inter: int = 2048
    n_shared: int = 1
    norm_eps: float = 1e-5
    expert_weights_norm: bool = True
    expert_weights_scale: float = 2.5
    dense_type: str = "q4_k"
    expert_type: str = "q2_k"

    @property
    def nope_dim(self) -> int:
        return self.key_mla_dim - self.rope_dim

    @classmethod
    def tiny(cls) -> "GLMDSAConfig":
        return cls(vocab_size=512, dim=256, n_layers=3, leading_dense_layers=1, n_heads=4, q_lora_rank=256, kv_lora_rank=256,
                   key_mla_dim=192, value_mla_dim=128, rope_dim=64, indexer_heads=4, indexer_key_dim=128, dsa_topk=8,
                   dense_inter=512, n_experts=8, top_k=2, expert_inter=256)

    def metadata(self) -> dict:
        p = ARCH + "."
        return {"general.architecture": ARCH, p + "vocab_size": self.vocab_size, p + "embedding_length": self.dim,
                p + "block_count": self.n_layers, p + "leading_dense_block_count": self.leading_dense_layers,
                p + "attention.head_count": self.n_heads, p + "attention.q_lora_rank": self.q_lora_rank,
                p + "attention.kv_lora_rank": self.kv_lora_rank, p + "attention.key_length_mla": self.key_mla_dim,
                p + "attention.value_length_mla": self.value_mla_dim, p + "rope.dimension_count": self.rope_dim,
                p + "rope.freq_base": float(self.rope_theta), p + "attention.indexer.head_count": self.indexer_heads,
                p + "attention.indexer.key_length": self.indexer_key_dim, p + "attention.indexer.top_k": self.dsa_topk,
                p + "feed_forward_length": self.dense_inter, p + "expert_count": self.n_experts, p + "expert_used_count": self.top_k,
                p + "expert_feed_forward_length": self.expert_inter, p + "expert_shared_count": self.n_shared,
                p + "attention.layer_norm_rms_epsilon": float(self.norm_eps), p + "expert_weights_norm": self.expert_weights_norm,
                p + "expert_weights_scale": float(self.expert_weights_scale)}

    @classmethod
    def from_gguf(cls, md: dict) -> "GLMDSAConfig":
        p = ARCH + "."
        g = lambda k, d=0: md.get(p + k, d)
        return cls(vocab_size=int(g("vocab_size", len(md.get("tokenizer.ggml.tokens", [])) or 154880)), dim=int(g("embedding_length")),
                   n_layers=int(g("block_count")) - int(g("nextn_predict_layers", 0)), leading_dense_layers=int(g("leading_dense_block_count", 0)),
                   n_heads=int(g("attention.head_count")), q_lora_rank=int(g("attention.q_lora_rank")),
                   kv_lora_rank=int(g("attention.kv_lora_rank")), key_mla_dim=int(g("attention.key_length_mla")),
                   value_mla_dim=int(g("attention.value_length_mla")), rope_dim=int(g("rope.dimension_count", 64)),
                   rope_theta=float(g("rope.freq_base", 1e6)), indexer_heads=int(g("attention.indexer.head_count", 0)),
                   indexer_key_dim=int(g("attention.indexer.key_length", 128)), dsa_topk=int(g("attention.indexer.top_k", 2048)),
                   dense_inter=int(g("feed_forward_length")), n_experts=int(g("expert_count")), top_k=int(g("expert_used_count")),
                   expert_inter=int(g("expert_feed_forward_length")), n_shared=int(g("expert_shared_count", 1)),
                   norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)), expert_weights_norm=bool(g("expert_weights_norm", False)),
                   expert_weights_scale=float(g("expert_weights_scale", 1.0)))


def tensor_plan(c: GLMDSAConfig) -> list[tuple[str, tuple[int, ...], str]]:
    H = c.dim
    out = [("token_embd.weight", (c.vocab_size, H), c.dense_type), ("output_norm.weight", (H,), "f32"),
           ("output.weight", (c.vocab_size, H), c.dense_type)]
    for i in range(c.n_layers):
        b = f"blk.{i}."
        out += [(b + "attn_norm.weight", (H,), "f32"), (b + "ffn_norm.weight", (H,), "f32"),
                (b + "attn_q_a.weight", (c.q_lora_rank, H), c.dense_type), (b + "attn_q_a_norm.weight", (c.q_lora_rank,), "f32"),
                (b + "attn_q_b.weight", (c.n_heads * c.key_mla_dim, c.q_lora_rank), c.dense_type),
                (b + "attn_kv_a_mqa.weight", (c.kv_lora_rank + c.rope_dim, H), "q8_0"), (b + "attn_kv_a_norm.weight", (c.kv_lora_rank,), "f32"),
                (b + "attn_k_b.weight", (c.n_heads, c.nope_dim, c.kv_lora_rank), "f32"),
                (b + "attn_v_b.weight", (c.n_heads, c.value_mla_dim, c.kv_lora_rank), "f32"),
                (b + "attn_output.weight", (H, c.n_heads * c.value_mla_dim), c.dense_type),
                (b + "indexer.attn_q_b.weight", (c.indexer_heads * c.indexer_key_dim, c.q_lora_rank), c.dense_type),
                (b + "indexer.attn_k.weight", (c.indexer_key_dim, H), "q8_0"), (b + "indexer.k_norm.weight", (c.indexer_key_dim,), "f32"),
                (b + "indexer.k_norm.bias", (c.indexer_key_dim,), "f32"), (b + "indexer.proj.weight", (c.indexer_heads, H), "f32")]
        if i < c.leading_dense_layers:
            out += [(b + "ffn_gate.weight", (c.dense_inter, H), c.dense_type), (b + "ffn_up.weight", (c.dense_inter, H), c.dense_type),
                    (b + "ffn_down.weight", (H, c.dense_inter), c.dense_type)]
        else:
            si = c.expert_inter * c.n_shared
            out += [(b + "ffn_gate_inp.weight", (c.n_experts, H), "f32"), (b + "exp_probs_b.bias", (c.n_experts,), "f32"),
                    (b + "ffn_gate_exps.weight", (c.n_experts, c.expert_inter, H), c.expert_type),
                    (b + "ffn_up_exps.weight", (c.n_experts, c.expert_inter, H), c.expert_type),
                    (b + "ffn_down_exps.weight", (c.n_experts, H, c.expert_inter), c.expert_type),
                    (b + "ffn_gate_shexp.weight", (si, H), c.dense_type), (b + "ffn_up_shexp.weight", (si, H), c.dense_type),
                    (b + "ffn_down_shexp.weight", (H, si), c.dense_type)]
    return out


def write_random_gguf(path: str | Path, cfg: GLMDSAConfig, seed: int = 0, sigma: float = 0.03) -> None:
    rng = np.random.default_rng(seed)
    w = gguf.GGUFWriter()
    for k, v in cfg.metadata().items():
        w.add_meta(k, v)
    for name, shape, typ in tensor_plan(cfg):
        if name.endswith("norm.weight"):
            data = (1.0 + 0.05 * rng.standard_normal(shape)).astype(np.float32)
        elif name.endswith(".bias"):
            data = (0.01 * rng.standard_normal(shape)).astype(np.float32)
        else:
            data = (sigma * rng.standard_normal(shape)).astype(np.float32)
        if typ == "f32":
            w.add_tensor(name, data, "f32", shape)
        else:
            w.add_tensor(name, gq.quantize(data, typ), typ, shape)
    w.write(path)


def rope_interleaved(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate pairs (2i, 2i+1) of the last dim. x [T, ..., R], pos [T]."""
    R = x.shape[-1]
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -torch.arange(0, R, 2, dtype=torch.float64) / R)
    ang = pos.double()[:, None] * inv.to(pos.device)[None, :]          # fp64 angles where `pos` lives: no host round trip
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [R // 2]
    cs, sn = torch.cos(ang).float().to(x.device).view(shape), torch.sin(ang).float().to(x.device).view(shape)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack([x0 * cs - x1 * sn, x0 * sn + x1 * cs], dim=-1).flatten(-2)


def _rms(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * g


def indexer_select(qi: torch.Tensor, ki: torch.Tensor, wh: torch.Tensor, pos: torch.Tensor, topk: int) -> torch.Tensor:
    """DSA lightning indexer. qi [T, Hi, Di], ki [S, Di] (all cached keys), wh [T, Hi] head
    weights, pos [T] absolute positions. Returns a bool mask [T, S] of the selected keys:
    the top-k scores among the causal positions (all of them when fewer than k exist);
    ties go to the lower position."""
    s = torch.relu(torch.einsum("thd,sd->ths", qi.float(), ki.float()))
    score = (s * wh.float()[:, :, None]).sum(1)                                   # [T, S]
    S = ki.shape[0]
    causal = torch.arange(S, device=qi.device)[None, :] <= pos[:, None]
    score = score.masked_fill(~causal, float("-inf"))
    if topk <= 0 or topk >= S:
        return causal
    mask = torch.zeros_like(causal)
    if score.is_cuda:
        # device radix select: the same set as the stable sort (ties to the lower position), -1 padded
        from ..ops import dsv4_ops as dk
        sel = dk.topk_select(score.contiguous(), topk).long()
        pad = torch.zeros(sel.shape[0], 1, dtype=torch.bool, device=sel.device)
        mask = torch.cat([mask, pad], 1).scatter_(1, torch.where(sel < 0, S, sel), True)[:, :S]
        return mask & causal
    # stable top-k: sort by (-score, position)
    order = torch.sort(-score, dim=-1, stable=True).indices[:, :topk]
    mask.scatter_(1, order, True)
    return mask & causal


class _Weights:
    """fp32 dequantised view of a checkpoint (oracle) or raw device blocks (runtime)."""

    def __init__(self, bundle: gguf.GGUFBundle):
        self.b = bundle

    def f32(self, name: str) -> torch.Tensor:
        t = self.b.info(name)
        src = self.b.raw(name) if t.type_name == "f32" else self.b.blocks(name)
        return torch.from_numpy(gq.dequantize(src, t.type_name).reshape(t.shape).copy())


class ReferenceModel:
    """fp32 PyTorch oracle (CPU, tiny shapes)."""

    def __init__(self, path: str | Path, dsa_topk: int | None = None):
        self.bundle = gguf.GGUFBundle(path)
        self.cfg = GLMDSAConfig.from_gguf(self.bundle.metadata)
        if dsa_topk is not None:
            self.cfg.dsa_topk = dsa_topk
        W = _Weights(self.bundle)
        self.w = {n: W.f32(n) for n in self.bundle.tensors}
        self.cache = [{"latent": [], "krope": [], "ki": []} for _ in range(self.cfg.n_layers)]
        self.pos = 0

    def forward(self, tokens: Sequence[int]) -> torch.Tensor:
        return _forward(self.cfg, self.w, self.cache, self, list(tokens), lambda x, name, **kw: _lin_f32(self.w, x, name, **kw))


def _lin_f32(w, x, name, gamma=None, eps=1e-5, swiglu_with=None):
    xf = x.float()
    if gamma is not None:
        xf = _rms(xf, gamma, eps).to(torch.bfloat16).float()
    if swiglu_with is not None:
        return (torch.nn.functional.silu(xf @ w[name].t()) * (xf @ w[swiglu_with].t())).to(torch.bfloat16)
    return (xf @ w[name].t())


def _forward(c: GLMDSAConfig, w: dict, cache: list, st, tokens: list[int], lin) -> torch.Tensor:
    """Shared model body: `lin(x, name, gamma=, swiglu_with=)` is the only backend-specific op."""
    dev = w["output_norm.weight"].device
    T = len(tokens)
    r16 = lambda t: t.to(torch.bfloat16).float()
    pos = torch.arange(st.pos, st.pos + T, device=dev)
    h = st.embed(tokens) if hasattr(st, "embed") else r16(w["token_embd.weight"][tokens])
    for i in range(c.n_layers):
        b = f"blk.{i}."
        an = w[b + "attn_norm.weight"]
        qa = r16(lin(h, b + "attn_q_a.weight", gamma=an, eps=c.norm_eps))
        qr = r16(_rms(qa, w[b + "attn_q_a_norm.weight"], c.norm_eps))
        q = r16(lin(qr, b + "attn_q_b.weight")).view(T, c.n_heads, c.key_mla_dim)
        kv = r16(lin(h, b + "attn_kv_a_mqa.weight", gamma=an, eps=c.norm_eps))
        latent = r16(_rms(kv[:, :c.kv_lora_rank], w[b + "attn_kv_a_norm.weight"], c.norm_eps))
        krope = r16(rope_interleaved(kv[:, c.kv_lora_rank:], pos, c.rope_theta))
        q = torch.cat([q[..., :c.nope_dim], r16(rope_interleaved(q[..., c.nope_dim:], pos, c.rope_theta))], dim=-1)
        # indexer keys / queries
        ki = lin(h, b + "indexer.attn_k.weight", gamma=an, eps=c.norm_eps).float()
        mu = ki.mean(-1, keepdim=True)
        ki = (ki - mu) * torch.rsqrt(((ki - mu) ** 2).mean(-1, keepdim=True) + c.norm_eps) * w[b + "indexer.k_norm.weight"] + w[b + "indexer.k_norm.bias"]
        ki = r16(torch.cat([rope_interleaved(ki[:, :c.rope_dim], pos, c.rope_theta), ki[:, c.rope_dim:]], dim=-1))
        qi = lin(qr, b + "indexer.attn_q_b.weight").float().view(T, c.indexer_heads, c.indexer_key_dim)
        qi = r16(torch.cat([rope_interleaved(qi[..., :c.rope_dim], pos, c.rope_theta), qi[..., c.rope_dim:]], dim=-1))
        xn = _rms(h.float(), an, c.norm_eps).to(torch.bfloat16).float()
        wh = (xn @ w[b + "indexer.proj.weight"].t()) * (c.indexer_heads * c.indexer_key_dim) ** -0.5
        cc = cache[i]
        cc["latent"].append(latent), cc["krope"].append(krope), cc["ki"].append(ki)
        LAT, KR, KI = torch.cat(cc["latent"]), torch.cat(cc["krope"]), torch.cat(cc["ki"])
        mask = indexer_select(qi, KI, wh, pos, c.dsa_topk)                          # [T, S]
        # absorbed MLA: scores on the latent, values from the latent
        q_lat = torch.einsum("thn,hnl->thl", q[..., :c.nope_dim], w[b + "attn_k_b.weight"])
        s = (torch.einsum("thl,sl->ths", q_lat, LAT) + torch.einsum("thr,sr->ths", q[..., c.nope_dim:], KR)) * c.key_mla_dim ** -0.5
        s = s.masked_fill(~mask[:, None, :], float("-inf"))
        o_lat = torch.einsum("ths,sl->thl", torch.softmax(s, -1), LAT)
        o = r16(torch.einsum("thl,hvl->thv", o_lat, w[b + "attn_v_b.weight"]).reshape(T, -1))
        h = r16(h + lin(o, b + "attn_output.weight").float())
        fn = w[b + "ffn_norm.weight"]
        if i < c.leading_dense_layers:
            mid = lin(h, b + "ffn_gate.weight", gamma=fn, eps=c.norm_eps, swiglu_with=b + "ffn_up.weight")
            h = r16(h + lin(mid, b + "ffn_down.weight").float())
        else:
            xn = _rms(h.float(), fn, c.norm_eps).to(torch.bfloat16)
            y = st.moe(i, xn)
            sh = lin(h, b + "ffn_gate_shexp.weight", gamma=fn, eps=c.norm_eps, swiglu_with=b + "ffn_up_shexp.weight")
            h = r16(h + y + lin(sh, b + "ffn_down_shexp.weight").float())
    st.pos += T
    return lin(h[-1:], "output.weight", gamma=w["output_norm.weight"], eps=c.norm_eps).float()[0]


def _moe_ref(self, i: int, xn: torch.Tensor) -> torch.Tensor:
    c, w, b = self.cfg, self.w, f"blk.{i}."
    x = xn.float()
    p = torch.sigmoid(x @ w[b + "ffn_gate_inp.weight"].t())
    ids = torch.topk(p + w[b + "exp_probs_b.bias"], c.top_k, dim=-1).indices
    wt = torch.gather(p, 1, ids)
    if c.expert_weights_norm:
        wt = wt / wt.sum(-1, keepdim=True)
    wt = wt * c.expert_weights_scale
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(c.top_k):
            e = int(ids[t, j])
            g, u = w[b + "ffn_gate_exps.weight"][e] @ x[t], w[b + "ffn_up_exps.weight"][e] @ x[t]
            y[t] += wt[t, j] * (w[b + "ffn_down_exps.weight"][e] @ (torch.nn.functional.silu(g) * u))
    return y


ReferenceModel.moe = _moe_ref


def _mla_attn(qk: torch.Tensor, kv_cache: torch.Tensor, pos: torch.Tensor, sel: torch.Tensor | None, scale: float) -> torch.Tensor:
    """Latent attention of bf16 q rows [T, H, D] over the position-indexed cache [ctx, D] (K row = V row): the rows `sel`
    names (int32 [T, k], -1 padded), or every row up to the query's position; bf16 [T, H, D]."""
    from ctypes import c_float, c_int
    from ..ops import _check, _ptr, _stream
    from ..ops import lib as _lib
    T, H, D = qk.shape
    out = torch.empty_like(qk)
    st = _lib.kernels().pk_dsv4_sparse_attn_ex(_ptr(qk), _ptr(kv_cache), _ptr(pos), _ptr(None), _ptr(sel), _ptr(None), _ptr(None), _ptr(None), c_int(T),
                                            c_int(H), c_int(D), c_int(0), c_int(0), c_int(1), c_int(2 if sel is not None else 1),
                                            c_int(0 if sel is None else sel.shape[1]), c_int(0), c_float(scale), _ptr(out), _stream())
    _check(st, "pk_dsv4_sparse_attn")
    return out


class GLMDSAModel:
    """GPU runtime: projections and experts on raw blocks; position-indexed latent and indexer-key caches allocated once; the
    lightning indexer through the index-score kernel and the device radix select, absorbed MLA attention through the
    latent sparse-attention kernel (`_forward_kernels`). Shapes the kernels do not take (indexer key dim other than 128,
    latent + rope width outside 128 / 320 / 512 / 576) run the shared PyTorch body."""

    def __init__(self, path: str | Path, *, device: str = "cuda", rank: int = 0, world: int = 1, max_context: int = 4096,
                 layers: int | None = None, group=None, dsa_topk: int | None = None, routed_tp: bool = False,
                 expert_slots: int | None = None, gpu_memory_gib: float | None = None):
        """`expert_slots` (or `gpu_memory_gib`, from which the slots per layer are planned): the routed experts of this
        rank stay in pinned host memory and only that many per layer are resident in HBM; a step's experts are staged on a
        side stream into least-recently-used slots (`moe.expert_cache.ExpertStagingCache`), steps that need more distinct
        experts than slots run in waves. For models whose experts exceed HBM.
        `routed_tp`: with several ranks, every rank keeps ALL experts but only its slice of the expert intermediate
        dimension (gate / up rows and the matching block columns of down, slices aligned to the 256-weight block), and the
        ranks' partial outputs are summed; the default splits whole experts over the ranks. (Reference: GLM_ROUTED_TP,
        src/models/glm_dsa/architecture.py:528-877, tests/test_glm_dsa_tp_routed.py.)"""
        from ..ops import gguf_ops as go
        self.go = go
        self.bundle = gguf.GGUFBundle(path)
        if self.bundle.architecture() != ARCH:
            raise ValueError(f"not a {ARCH} checkpoint")
        self.cfg = c = GLMDSAConfig.from_gguf(self.bundle.metadata)
        if layers:
            c.n_layers = min(c.n_layers, layers)
        if dsa_topk is not None:
            c.dsa_topk = dsa_topk
        if c.n_experts % world:
            raise ValueError("expert count must divide by the world size")
        self.device, self.rank, self.world, self.group = torch.device(device), rank, world, group
        self.e_local, self.e_start = c.n_experts // world, rank * (c.n_experts // world)
        self.routed_tp = bool(routed_tp) and world > 1
        self.inter_local = c.expert_inter
        if self.routed_tp:
            if c.expert_inter % (256 * world):
                raise ValueError("routed TP needs the expert intermediate size to be a multiple of 256 * world (block-aligned slices)")
            self.e_local, self.e_start = c.n_experts, 0
            self.inter_local = c.expert_inter // world
        self._combiner = None
        self.types = {n: t.type_name for n, t in self.bundle.tensors.items()}
        self.shapes = {n: t.shape for n, t in self.bundle.tensors.items()}
        W = _Weights(self.bundle)
        self.w: dict[str, torch.Tensor] = {}    # fp32 small tensors
        self.raw: dict[str, torch.Tensor] = {}  # raw blocks
        keep = [f"blk.{i}." for i in range(c.n_layers)]
        n_moe = c.n_layers - c.leading_dense_layers
        if expert_slots is None and gpu_memory_gib is not None and n_moe > 0:
            from ..moe.expert_cache import slots_for_budget
            exp_names = [n for n in self.bundle.tensors if n.startswith(f"blk.{c.leading_dense_layers}.") and "_exps." in n]
            per_expert = sum(int(self.bundle.tensors[n].nbytes) // c.n_experts for n in exp_names) // (world if self.routed_tp else 1)
            other = sum(int(t.nbytes) for n, t in self.bundle.tensors.items()
                        if "_exps." not in n and (not n.startswith("blk.") or any(n.startswith(k) for k in keep)))
            kv = c.n_layers * max_context * (c.kv_lora_rank + c.rope_dim + c.indexer_key_dim) * 2
            budget = int(gpu_memory_gib * (1 << 30)) - other - kv - (2 << 30)        # 2 GiB for activations, scratch and the context
            expert_slots = slots_for_budget(max(budget, 0), per_expert, n_moe, self.e_local, c.top_k)
        staged = expert_slots is not None and expert_slots < self.e_local
        self.expert_slots = expert_slots if staged else None
        for n, t in self.bundle.tensors.items():
            if n.startswith("blk.") and not any(n.startswith(k) for k in keep):
                continue
            if t.type_name == "f32":
                self.w[n] = W.f32(n).to(self.device)
            elif "_exps." in n:
                blk = self.bundle.blocks(n)[self.e_start:self.e_start + self.e_local]       # [experts, rows, blocks per row, block bytes]
                if self.routed_tp:
                    il = self.inter_local
                    if "ffn_down_exps" in n:                                             # K slice: whole 256-weight blocks of every row
                        blk = blk[:, :, rank * il // 256:(rank + 1) * il // 256]
                    else:                                                                # gate / up: this rank's rows
                        blk = blk[:, rank * il:(rank + 1) * il]
                t_host = torch.from_numpy(np.ascontiguousarray(blk).reshape(self.e_local, -1))
                self.raw[n] = t_host if staged else t_host.to(self.device)
            else:
                self.raw[n] = torch.from_numpy(np.ascontiguousarray(self.bundle.blocks(n)).reshape(-1)).to(self.device)
        for i in range(c.leading_dense_layers, c.n_layers):
            b = f"blk.{i}."
            self.raw[b + "w13"] = torch.cat([self.raw.pop(b + "ffn_gate_exps.weight"), self.raw.pop(b + "ffn_up_exps.weight")], dim=1).contiguous()
        self.staging: dict[int, object] = {}
        if staged:
            from ..moe.expert_cache import ExpertStagingCache
            for i in range(c.leading_dense_layers, c.n_layers):
                b = f"blk.{i}."
                # the host copies move to pinned memory inside the cache; HBM holds `expert_slots` experts per layer
                self.staging[i] = ExpertStagingCache({"w13": self.raw.pop(b + "w13"), "w2": self.raw.pop(b + "ffn_down_exps.weight")},
                                                     slots=expert_slots, device=self.device)
        self.cache = [{"latent": [], "krope": [], "ki": []} for _ in range(c.n_layers)]
        self.max_context, self.pos = max_context, 0

    def _combine(self, y: torch.Tensor) -> torch.Tensor:
        """Sum the ranks' expert outputs (peer-memory all-reduce for small payloads, NCCL for large ones)."""
        if self._combiner is None:
            from ..parallel.combine import ExpertCombine
            self._combiner = ExpertCombine(self.world, self.group)
        return self._combiner(y)

    def reset(self) -> None:
        self.pos = 0
        for cc in self.cache:
            cc["latent"].clear(), cc["krope"].clear(), cc["ki"].clear()

    def embed(self, tokens: list[int]) -> torch.Tensor:
        t = torch.tensor(tokens, dtype=torch.int32, device=self.device)
        return self.go.gguf_dequant_rows(self.raw["token_embd.weight"], self.types["token_embd.weight"], self.cfg.dim, t).float()

    def _lin(self, x: torch.Tensor, name: str, gamma=None, eps=1e-5, swiglu_with=None) -> torch.Tensor:
        go, xb = self.go, x.to(torch.bfloat16).contiguous()
        N = self.shapes[name][0]
        if swiglu_with is not None:
            g = go.gguf_linear(xb, self.raw[name], self.types[name], N, gamma=gamma, eps=eps, epi=2)
            u = go.gguf_linear(xb, self.raw[swiglu_with], self.types[swiglu_with], N, gamma=gamma, eps=eps, epi=2)
            return (torch.nn.functional.silu(g) * u).to(torch.bfloat16)
        return go.gguf_linear(xb, self.raw[name], self.types[name], N, gamma=gamma, eps=eps, epi=2)

    def moe(self, i: int, xn: torch.Tensor) -> torch.Tensor:
        c, go, b = self.cfg, self.go, f"blk.{i}."
        xb = xn.to(torch.bfloat16).contiguous()
        ids, wt = go.router_topk(xb, self.w[b + "ffn_gate_inp.weight"], c.top_k, bias=self.w[b + "exp_probs_b.bias"],
                                 score_func="sigmoid", norm_topk=c.expert_weights_norm, route_scale=c.expert_weights_scale)
        if i in self.staging:
            from ..moe.expert_cache import staged_moe_forward
            # routes to other ranks' experts become weight-0 routes to this rank's first expert: they add exactly nothing
            mine = (ids >= self.e_start) & (ids < self.e_start + self.e_local)
            ids_l = torch.where(mine, ids - self.e_start, torch.zeros_like(ids)).contiguous()
            wt_l = torch.where(mine, wt, torch.zeros_like(wt)).contiguous()
            y = staged_moe_forward(self.staging[i], xb, ids_l, wt_l, self.types[b + "ffn_gate_exps.weight"],
                                   self.types[b + "ffn_down_exps.weight"], self.inter_local)
            if self.world > 1:
                self._combine(y)
            return y
        routes = go.group_routes(ids, wt, c.n_experts)
        y = go.moe_forward(xb, self.raw[b + "w13"], self.raw[b + "ffn_down_exps.weight"], self.types[b + "ffn_gate_exps.weight"],
                           self.types[b + "ffn_down_exps.weight"], c.n_experts, self.inter_local, routes,
                           expert_offset=self.e_start, local_experts=self.e_local)
        if self.world > 1:
            self._combine(y)
        return y

    def _kernel_attention_ok(self) -> bool:
        c = self.cfg
        return c.indexer_key_dim == 128 and (c.kv_lora_rank + c.rope_dim) in (128, 320, 512, 576)

    def _alloc_kernel_caches(self) -> None:
        c = self.cfg
        self.kv_cache = [torch.zeros(self.max_context, c.kv_lora_rank + c.rope_dim, device=self.device, dtype=torch.bfloat16) for _ in range(c.n_layers)]
        self.ki_cache = [torch.zeros(self.max_context, c.indexer_key_dim, device=self.device, dtype=torch.bfloat16) for _ in range(c.n_layers)]

    @torch.no_grad()
    def forward(self, tokens: Sequence[int]) -> torch.Tensor:
        if self.pos + len(tokens) > self.max_context:
            raise ValueError("context exceeds max_context")
        if not self._kernel_attention_ok():
            return _forward(self.cfg, self.w, self.cache, self, list(tokens), self._lin)
        return self._forward_kernels(list(tokens))

    @torch.no_grad()
    def _forward_kernels(self, tokens: list[int]) -> torch.Tensor:
        """The model body on the framework's kernels: raw-block linears, position-indexed latent / rope and indexer-key caches
        allocated once (nothing is concatenated per step), the lightning indexer as the index-score kernel + device radix
        select, and absorbed MLA attention as the sparse-attention kernel over the latent cache (a key row is
        [latent | rotated rope part], the value is its latent part). Same numerics as `_forward` (the oracle's body)."""
        from ..ops import dsv4_ops as dk
        c, w, lin = self.cfg, self.w, self._lin
        if not hasattr(self, "kv_cache"):
            self._alloc_kernel_caches()
        T, dev = len(tokens), self.device
        r16 = lambda t: t.to(torch.bfloat16).float()
        p0 = self.pos
        pos = torch.arange(p0, p0 + T, device=dev)
        pos32 = pos.to(torch.int32)
        S = p0 + T
        h = self.embed(tokens)
        L, R = c.kv_lora_rank, c.rope_dim
        for i in range(c.n_layers):
            b = f"blk.{i}."
            an = w[b + "attn_norm.weight"]
            qa = r16(lin(h, b + "attn_q_a.weight", gamma=an, eps=c.norm_eps))
            qr = r16(_rms(qa, w[b + "attn_q_a_norm.weight"], c.norm_eps))
            q = r16(lin(qr, b + "attn_q_b.weight")).view(T, c.n_heads, c.key_mla_dim)
            kv = r16(lin(h, b + "attn_kv_a_mqa.weight", gamma=an, eps=c.norm_eps))
            latent = _rms(kv[:, :L], w[b + "attn_kv_a_norm.weight"], c.norm_eps)
            krope = rope_interleaved(kv[:, L:], pos, c.rope_theta)
            self.kv_cache[i][p0:S] = torch.cat([latent, krope], -1).to(torch.bfloat16)
            q_rope = r16(rope_interleaved(q[..., c.nope_dim:], pos, c.rope_theta))
            # indexer keys of the new rows
            ki = lin(h, b + "indexer.attn_k.weight", gamma=an, eps=c.norm_eps).float()
            mu = ki.mean(-1, keepdim=True)
            ki = (ki - mu) * torch.rsqrt(((ki - mu) ** 2).mean(-1, keepdim=True) + c.norm_eps) * w[b + "indexer.k_norm.weight"] + w[b + "indexer.k_norm.bias"]
            ki = torch.cat([rope_interleaved(ki[:, :R], pos, c.rope_theta), ki[:, R:]], dim=-1)
            self.ki_cache[i][p0:S] = ki.to(torch.bfloat16)
            sel = None
            if 0 < c.dsa_topk < S:
                qi = lin(qr, b + "indexer.attn_q_b.weight").float().view(T, c.indexer_heads, c.indexer_key_dim)
                qi = torch.cat([rope_interleaved(qi[..., :R], pos, c.rope_theta), qi[..., R:]], dim=-1).to(torch.bfloat16).contiguous()
                xn = _rms(h.float(), an, c.norm_eps).to(torch.bfloat16).float()
                wh = (xn @ w[b + "indexer.proj.weight"].t()).contiguous()
                score = dk.index_score(qi, self.ki_cache[i], wh, pos32, 1, S, (c.indexer_heads * c.indexer_key_dim) ** -0.5)
                sel = dk.topk_select(score, c.dsa_topk)                   # positions a row cannot see score -inf and are never picked
            # absorbed MLA: q against [latent | rope] rows, output in latent space
            q_lat = torch.einsum("thn,hnl->thl", q[..., :c.nope_dim], w[b + "attn_k_b.weight"])
            qk = torch.cat([q_lat, q_rope], -1).to(torch.bfloat16).contiguous()
            o_lat = _mla_attn(qk, self.kv_cache[i], pos32, sel, c.key_mla_dim ** -0.5)[..., :L].float()
            o = r16(torch.einsum("thl,hvl->thv", o_lat, w[b + "attn_v_b.weight"]).reshape(T, -1))
            h = r16(h + lin(o, b + "attn_output.weight").float())
            fn = w[b + "ffn_norm.weight"]
            if i < c.leading_dense_layers:
                mid = lin(h, b + "ffn_gate.weight", gamma=fn, eps=c.norm_eps, swiglu_with=b + "ffn_up.weight")
                h = r16(h + lin(mid, b + "ffn_down.weight").float())
            else:
                xn = _rms(h.float(), fn, c.norm_eps).to(torch.bfloat16)
                y = self.moe(i, xn)
                sh = lin(h, b + "ffn_gate_shexp.weight", gamma=fn, eps=c.norm_eps, swiglu_with=b + "ffn_up_shexp.weight")
                h = r16(h + y + lin(sh, b + "ffn_down_shexp.weight").float())
        self.pos += T
        return lin(h[-1:], "output.weight", gamma=w["output_norm.weight"], eps=c.norm_eps).float()[0]

    def _checked(self, token: int) -> int:
        """The step's token, or `StepFailed` on every rank when a peer all-reduce timed out (collective check)."""
        if self._combiner is not None:
            self._combiner.check_step(self.device)
        return token

    def forward_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """fp32 logits after feeding `tokens` at the current position (for host-side sampling and log-probabilities)."""
        return self.forward(tokens)

    def prefill(self, tokens: Sequence[int]) -> int:
        return self._checked(int(torch.argmax(self.forward(tokens))))

    def decode_one(self, token: int) -> int:
        return self._checked(int(torch.argmax(self.forward([token]))))
