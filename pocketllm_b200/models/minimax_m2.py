"""MiniMax-M2 on raw GGUF blocks: GQA attention + sigmoid top-k routed MoE, no shared expert.

Numerical contract (reference: src/models/minimax_m2/architecture.py:57-472): plain-gamma
RMSNorm; q/k norms over the whole projected vector; half-split RoPE on the first
`rope_dim` dims; softmax scale 1/sqrt(head_dim); router p = sigmoid(x W^T), top-k of p + bias,
weights p normalised to sum 1; experts are SwiGLU. Attention weights are Q5_K, embedding and
output Q4_K, experts IQ2_XXS (other mixes: Q2_K, IQ1_M).

Execution here: every projection and expert runs on the raw blocks (`ops.gguf_ops`), the
attention core on the split-context GQA kernel, experts are partitioned over ranks
(contiguous ranges) and the per-token outputs are summed across ranks.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

import numpy as np
import torch

from ..formats import gguf, gguf_quants as gq

ARCH = "minimax-m2"


@dataclass
class MiniMaxM2Config:
    vocab_size: int = 200064
    dim: int = 3072
    n_layers: int = 62
    n_heads: int = 48
    n_kv_heads: int = 8
    head_dim: int = 128
    rope_dim: int = 64
    rope_theta: float = 5.0e6
    n_experts: int = 256
    n_experts_used: int = 8
    expert_inter: int = 1536
    norm_eps: float = 1e-6
    attn_type: str = "q5_k"
    embed_type: str = "q4_k"
    expert_type: str = "iq2_xxs"
    expert_down_type: str = "iq2_xxs"

    @classmethod
    def from_gguf(cls, md: dict) -> "MiniMaxM2Config":
        p = ARCH + "."
        return cls(vocab_size=int(md.get(p + "vocab_size", len(md.get("tokenizer.ggml.tokens", [])) or 200064)),
                   dim=int(md[p + "embedding_length"]), n_layers=int(md[p + "block_count"]),
                   n_heads=int(md[p + "attention.head_count"]), n_kv_heads=int(md[p + "attention.head_count_kv"]),
                   head_dim=int(md.get(p + "attention.key_length", 128)), rope_dim=int(md.get(p + "rope.dimension_count", 64)),
                   rope_theta=float(md.get(p + "rope.freq_base", 5e6)), n_experts=int(md[p + "expert_count"]),
                   n_experts_used=int(md[p + "expert_used_count"]), expert_inter=int(md[p + "expert_feed_forward_length"]),
                   norm_eps=float(md.get(p + "attention.layer_norm_rms_epsilon", 1e-6)))

    @classmethod
    def tiny(cls) -> "MiniMaxM2Config":
        return cls(vocab_size=512, dim=256, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128, rope_dim=64, n_experts=8,
                   n_experts_used=2, expert_inter=256)

    def metadata(self) -> dict:
        p = ARCH + "."
        return {"general.architecture": ARCH, p + "vocab_size": self.vocab_size, p + "embedding_length": self.dim,
                p + "block_count": self.n_layers, p + "attention.head_count": self.n_heads,
                p + "attention.head_count_kv": self.n_kv_heads, p + "attention.key_length": self.head_dim,
                p + "rope.dimension_count": self.rope_dim, p + "rope.freq_base": float(self.rope_theta),
                p + "expert_count": self.n_experts, p + "expert_used_count": self.n_experts_used,
                p + "expert_feed_forward_length": self.expert_inter, p + "attention.layer_norm_rms_epsilon": float(self.norm_eps)}


def tensor_plan(cfg: MiniMaxM2Config) -> list[tuple[str, tuple[int, ...], str]]:
    """(name, logical shape, ggml type) of every tensor of the checkpoint."""
    H, D = cfg.dim, cfg.head_dim
    out = [("token_embd.weight", (cfg.vocab_size, H), cfg.embed_type), ("output_norm.weight", (H,), "f32"),
           ("output.weight", (cfg.vocab_size, H), cfg.embed_type)]
    for i in range(cfg.n_layers):
        b = f"blk.{i}."
        out += [(b + "attn_norm.weight", (H,), "f32"), (b + "ffn_norm.weight", (H,), "f32"),
                (b + "attn_q.weight", (cfg.n_heads * D, H), cfg.attn_type), (b + "attn_k.weight", (cfg.n_kv_heads * D, H), cfg.attn_type),
                (b + "attn_v.weight", (cfg.n_kv_heads * D, H), cfg.attn_type), (b + "attn_output.weight", (H, cfg.n_heads * D), cfg.attn_type),
                (b + "attn_q_norm.weight", (cfg.n_heads * D,), "f32"), (b + "attn_k_norm.weight", (cfg.n_kv_heads * D,), "f32"),
                (b + "ffn_gate_inp.weight", (cfg.n_experts, H), "f32"), (b + "exp_probs_b.bias", (cfg.n_experts,), "f32"),
                (b + "ffn_gate_exps.weight", (cfg.n_experts, cfg.expert_inter, H), cfg.expert_type),
                (b + "ffn_up_exps.weight", (cfg.n_experts, cfg.expert_inter, H), cfg.expert_type),
                (b + "ffn_down_exps.weight", (cfg.n_experts, H, cfg.expert_inter), cfg.expert_down_type)]
    return out


def write_random_gguf(path: str | Path, cfg: MiniMaxM2Config, seed: int = 0, sigma: float = 0.02) -> None:
    """Random-init checkpoint with real block payloads (N(0, sigma) through the quantisers)."""
    rng = np.random.default_rng(seed)
    w = gguf.GGUFWriter()
    for k, v in cfg.metadata().items():
        w.add_meta(k, v)
    for name, shape, typ in tensor_plan(cfg):
        if typ == "f32":
            if name.endswith("norm.weight"):
                data = (1.0 + 0.05 * rng.standard_normal(shape)).astype(np.float32)
            else:
                data = (sigma * rng.standard_normal(shape)).astype(np.float32)
            w.add_tensor(name, data, "f32", shape)
        else:
            x = (sigma * rng.standard_normal(shape)).astype(np.float32)
            w.add_tensor(name, gq.quantize(x, typ), typ, shape)
    w.write(path)


def _rope(x: torch.Tensor, pos: torch.Tensor, rope_dim: int, theta: float) -> torch.Tensor:
    """Half-split rotation of the first rope_dim dims. x [T, heads, D], pos [T]."""
    half = rope_dim // 2
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rope_dim)
    ang = pos.double().cpu()[:, None] * inv[None, :]
    cs, sn = torch.cos(ang).float().to(x.device)[:, None, :], torch.sin(ang).float().to(x.device)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:rope_dim]
    return torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn, x[..., rope_dim:]], dim=-1)


def _rope_tables(max_context: int, rope_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [max_context, rope_dim / 2] in fp32 from fp64 angles (what `_rope` computes per call on the host)."""
    half = rope_dim // 2
    inv = torch.pow(torch.tensor(theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rope_dim)
    ang = torch.arange(max_context, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cos(ang).float().to(device), torch.sin(ang).float().to(device)


def _rope_lookup(x: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor, rope_dim: int) -> torch.Tensor:
    """`_rope` with the angles taken from device tables: no host round trip, usable under stream capture."""
    half = rope_dim // 2
    idx = pos.long()
    cs, sn = cos_t[idx][:, None, :], sin_t[idx][:, None, :]
    x1, x2 = x[..., :half], x[..., half:rope_dim]
    return torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn, x[..., rope_dim:]], dim=-1)


def _rms(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * g


class ReferenceModel:
    """fp32 PyTorch oracle on dequantised weights (CPU, tiny shapes)."""

    def __init__(self, path: str | Path):
        self.bundle = gguf.GGUFBundle(path)
        self.cfg = MiniMaxM2Config.from_gguf(self.bundle.metadata)
        self.w = {n: torch.from_numpy(gq.dequantize(self.bundle.blocks(n) if t.type_name not in ("f32",) else self.bundle.raw(n),
                                                    t.type_name).reshape(t.shape).copy())
                  for n, t in self.bundle.tensors.items()}
        self.k: list[list[torch.Tensor]] = [[] for _ in range(self.cfg.n_layers)]
        self.v: list[list[torch.Tensor]] = [[] for _ in range(self.cfg.n_layers)]
        self.pos = 0

    def forward(self, tokens: Sequence[int]) -> torch.Tensor:
        c, w = self.cfg, self.w
        T = len(tokens)
        r16 = lambda t: t.to(torch.bfloat16).float()
        pos = torch.arange(self.pos, self.pos + T)
        h = r16(w["token_embd.weight"][list(tokens)])
        for i in range(c.n_layers):
            b = f"blk.{i}."
            x = r16(_rms(h, w[b + "attn_norm.weight"], c.norm_eps))
            q, k, v = r16(x @ w[b + "attn_q.weight"].t()), r16(x @ w[b + "attn_k.weight"].t()), r16(x @ w[b + "attn_v.weight"].t())
            q = _rms(q, w[b + "attn_q_norm.weight"], c.norm_eps).view(T, c.n_heads, c.head_dim)
            k = _rms(k, w[b + "attn_k_norm.weight"], c.norm_eps).view(T, c.n_kv_heads, c.head_dim)
            q, k = r16(_rope(q, pos, c.rope_dim, c.rope_theta)), r16(_rope(k, pos, c.rope_dim, c.rope_theta))
            self.k[i].append(k)
            self.v[i].append(v.view(T, c.n_kv_heads, c.head_dim))
            K, V = torch.cat(self.k[i]), torch.cat(self.v[i])
            rep = c.n_heads // c.n_kv_heads
            K, V = K.repeat_interleave(rep, 1), V.repeat_interleave(rep, 1)
            s = torch.einsum("thd,shd->hts", q, K) * c.head_dim ** -0.5
            mask = torch.arange(K.shape[0])[None, :] > pos[:, None]
            s = s.masked_fill(mask[None], float("-inf"))
            o = r16(torch.einsum("hts,shd->thd", torch.softmax(s, -1), V).reshape(T, -1))
            h = r16(h + o @ w[b + "attn_output.weight"].t())
            x = r16(_rms(h, w[b + "ffn_norm.weight"], c.norm_eps))
            p = torch.sigmoid(x @ w[b + "ffn_gate_inp.weight"].t())
            ids = torch.topk(p + w[b + "exp_probs_b.bias"], c.n_experts_used, dim=-1).indices
            wt = torch.gather(p, 1, ids)
            wt = wt / wt.sum(-1, keepdim=True)
            y = torch.zeros_like(h)
            for t in range(T):
                for j in range(c.n_experts_used):
                    e = int(ids[t, j])
                    g, u = w[b + "ffn_gate_exps.weight"][e] @ x[t], w[b + "ffn_up_exps.weight"][e] @ x[t]
                    y[t] += wt[t, j] * (w[b + "ffn_down_exps.weight"][e] @ (torch.nn.functional.silu(g) * u))
            h = r16(h + y)
        self.pos += T
        x = r16(_rms(h, w["output_norm.weight"], c.norm_eps))
        return x @ w["output.weight"].t()


class MiniMaxM2Model:
    """GPU runtime on raw blocks. `expert range` of rank r: [r * E/W, (r+1) * E/W)."""

    def __init__(self, path: str | Path, *, device: str = "cuda", rank: int = 0, world: int = 1, max_context: int = 4096,
                 layers: int | None = None, group=None, expert_slots: int | None = None):
        """`expert_slots`: keep this rank's routed experts in pinned host memory and only that many per layer in HBM, staged
        on a side stream into least-recently-used slots (`moe.expert_cache.ExpertStagingCache`)."""
        from ..ops import gguf_ops as go
        self.go = go
        self.bundle = gguf.GGUFBundle(path)
        if self.bundle.architecture() != ARCH:
            raise ValueError(f"not a {ARCH} checkpoint: {self.bundle.architecture()!r}")
        self.cfg = c = MiniMaxM2Config.from_gguf(self.bundle.metadata)
        if layers:
            c.n_layers = min(c.n_layers, layers)
        if c.n_experts % world:
            raise ValueError("expert count must divide by the world size")
        self.device, self.rank, self.world, self.group = torch.device(device), rank, world, group
        self.e_local = c.n_experts // world
        self._combiner = None
        self.e_start = rank * self.e_local
        self.types = {n: t.type_name for n, t in self.bundle.tensors.items()}

        def raw(name: str, lo: int | None = None, hi: int | None = None) -> torch.Tensor:
            b = self.bundle.blocks(name)
            if lo is not None:
                b = b[lo:hi]
            return torch.from_numpy(np.array(b, copy=True).reshape(-1)).to(self.device)

        def f32(name: str) -> torch.Tensor:
            return torch.from_numpy(self.bundle.raw(name).view(np.float32).copy()).to(self.device)

        self.embed, self.head = raw("token_embd.weight"), raw("output.weight")
        self.final_norm = f32("output_norm.weight")
        self.layers = []
        for i in range(c.n_layers):
            b = f"blk.{i}."
            L = {"attn_norm": f32(b + "attn_norm.weight"), "ffn_norm": f32(b + "ffn_norm.weight"),
                 "q": raw(b + "attn_q.weight"), "k": raw(b + "attn_k.weight"), "v": raw(b + "attn_v.weight"),
                 "o": raw(b + "attn_output.weight"), "q_norm": f32(b + "attn_q_norm.weight"), "k_norm": f32(b + "attn_k_norm.weight"),
                 "router": f32(b + "ffn_gate_inp.weight").view(c.n_experts, c.dim), "bias": f32(b + "exp_probs_b.bias"),
                 # gate rows then up rows per expert, this rank's experts only
                 "w13": torch.cat([raw(b + "ffn_gate_exps.weight", self.e_start, self.e_start + self.e_local).view(self.e_local, -1),
                                   raw(b + "ffn_up_exps.weight", self.e_start, self.e_start + self.e_local).view(self.e_local, -1)], dim=1).contiguous(),
                 "w2": raw(b + "ffn_down_exps.weight", self.e_start, self.e_start + self.e_local),
                 "kc": torch.zeros(c.n_kv_heads, max_context, c.head_dim, device=self.device, dtype=torch.bfloat16),
                 "vc": torch.zeros(c.n_kv_heads, max_context, c.head_dim, device=self.device, dtype=torch.bfloat16)}
            self.layers.append(L)
        if expert_slots is not None and expert_slots < self.e_local:
            from ..moe.expert_cache import ExpertStagingCache
            for L in self.layers:
                L["cache"] = ExpertStagingCache({"w13": L.pop("w13").cpu(), "w2": L.pop("w2").view(self.e_local, -1).cpu()}, slots=expert_slots,
                                                device=self.device)
        self.max_context = max_context
        self.pos = 0
        self._finish_init()

    @classmethod
    def synthetic(cls, cfg: MiniMaxM2Config, *, device: str = "cuda", rank: int = 0, world: int = 1, max_context: int = 4096,
                  seed: int = 0, group=None) -> "MiniMaxM2Model":
        """A model of shape `cfg` whose quantised tensors are random block payloads made on the device (block scales set
        to a small constant so that every weight is finite): for timing full-size shapes that no file on disk provides.
        Only block types whose scale is a leading fp16 field are accepted (q4_k, q5_k, q8_0, iq2_xxs, iq2_xs, iq3_xxs)."""
        from ..ops import gguf_ops as go
        if cfg.n_experts % world:
            raise ValueError("expert count must divide by the world size")
        self = cls.__new__(cls)
        self.go, self.bundle, self.cfg = go, None, cfg
        self.device, self.rank, self.world, self.group = torch.device(device), rank, world, group
        self.e_local = cfg.n_experts // world
        self.e_start = rank * self.e_local
        self._combiner = None
        self.types = {n: t for n, _, t in tensor_plan(cfg)}
        g = torch.Generator(device=self.device).manual_seed(seed)             # replicated tensors: the same draw on every rank
        ge = torch.Generator(device=self.device).manual_seed(seed * 1000 + 17 + rank)
        scale_bytes = torch.tensor([0x00, 0x10], dtype=torch.uint8, device=self.device)   # fp16 2^-11
        n_scale_fields = {"q4_k": 2, "q5_k": 2, "q8_0": 1, "iq2_xxs": 1, "iq2_xs": 1, "iq3_xxs": 1}

        def blocks(typ: str, rows: int, K: int, gen) -> torch.Tensor:
            if typ not in n_scale_fields:
                raise ValueError(f"synthetic blocks of type {typ} are not supported")
            rb = go.row_bytes(typ, K)
            per_block = rb * (32 if typ == "q8_0" else 256) // K
            out = torch.empty(rows * rb, dtype=torch.uint8, device=self.device)
            step = max(1, (256 << 20) // rb)
            for r0 in range(0, rows, step):                                        # 256 MB at a time
                n = min(step, rows - r0) * rb
                out[r0 * rb: r0 * rb + n] = torch.randint(0, 256, (n,), dtype=torch.uint8, device=self.device, generator=gen)
            v = out.view(-1, per_block)
            for f in range(n_scale_fields[typ]):
                v[:, 2 * f: 2 * f + 2] = scale_bytes
            return out

        def f32(*shape, mean=0.0, std=0.02) -> torch.Tensor:
            return mean + std * torch.randn(*shape, device=self.device, generator=g)

        c = cfg
        D = c.head_dim
        self.embed = blocks(c.embed_type, c.vocab_size, c.dim, g)
        self.head = blocks(c.embed_type, c.vocab_size, c.dim, g)
        self.final_norm = f32(c.dim, mean=1.0, std=0.05)
        self.layers = []
        for i in range(c.n_layers):
            L = {"attn_norm": f32(c.dim, mean=1.0, std=0.05), "ffn_norm": f32(c.dim, mean=1.0, std=0.05),
                 "q": blocks(c.attn_type, c.n_heads * D, c.dim, g), "k": blocks(c.attn_type, c.n_kv_heads * D, c.dim, g),
                 "v": blocks(c.attn_type, c.n_kv_heads * D, c.dim, g), "o": blocks(c.attn_type, c.dim, c.n_heads * D, g),
                 "q_norm": f32(c.n_heads * D, mean=1.0, std=0.05), "k_norm": f32(c.n_kv_heads * D, mean=1.0, std=0.05),
                 "router": f32(c.n_experts, c.dim), "bias": f32(c.n_experts),
                 "w13": torch.cat([blocks(c.expert_type, self.e_local * c.expert_inter, c.dim, ge).view(self.e_local, -1),
                                   blocks(c.expert_type, self.e_local * c.expert_inter, c.dim, ge).view(self.e_local, -1)], dim=1).contiguous(),
                 "w2": blocks(c.expert_down_type, self.e_local * c.dim, c.expert_inter, ge),
                 "kc": torch.zeros(c.n_kv_heads, max_context, D, device=self.device, dtype=torch.bfloat16),
                 "vc": torch.zeros(c.n_kv_heads, max_context, D, device=self.device, dtype=torch.bfloat16)}
            self.layers.append(L)
        self.max_context = max_context
        self.pos = 0
        self._finish_init()
        return self

    def _finish_init(self) -> None:
        c = self.cfg
        for i, L in enumerate(self.layers):
            b = f"blk.{i}."
            if self.types[b + "attn_q.weight"] == self.types[b + "attn_k.weight"] == self.types[b + "attn_v.weight"]:
                L["qkv"] = torch.cat([L.pop("q"), L.pop("k"), L.pop("v")])       # raw rows are contiguous per tensor: row-wise concat
        self.rope_cos, self.rope_sin = _rope_tables(self.max_context, c.rope_dim, c.rope_theta, self.device)
        # single-token decode replays one captured CUDA graph: on by default on one rank (POCKET_GGUF_DECODE_GRAPH=0 turns
        # it off), opt-in with several ranks (=2: the expert combine is then captured too, all ranks replay in step)
        self.balanced_routes = False
        mode = os.environ.get("POCKET_GGUF_DECODE_GRAPH", "1")
        self.use_graph = self.device.type == "cuda" and (mode == "2" or (mode != "0" and self.world == 1))
        if any("cache" in L for L in self.layers):
            self.use_graph = False     # staged experts: which experts a step needs is read on the host
        self._graph = None

    def _combine(self, y: torch.Tensor) -> torch.Tensor:
        """Sum the ranks' expert outputs (peer-memory all-reduce for small payloads, NCCL for large ones)."""
        if self._combiner is None:
            from ..parallel.combine import ExpertCombine
            self._combiner = ExpertCombine(self.world, self.group)
        return self._combiner(y)

    def _peer(self):
        """The peer-memory context of the expert-parallel group (None on one rank or after the peer path was dropped): the
        grouped expert path finishes with its combine kernel instead of a separate all-reduce."""
        if self.world == 1:
            return None
        if self._combiner is None:
            from ..parallel.combine import ExpertCombine
            self._combiner = ExpertCombine(self.world, self.group)
        return self._combiner.peer

    def reset(self) -> None:
        self.pos = 0

    def weight_bytes(self) -> int:
        n = self.embed.numel() + self.head.numel()
        for L in self.layers:
            n += sum(L[k].numel() * L[k].element_size() for k in ("q", "k", "v", "qkv", "o", "w13", "w2", "router") if k in L)
        return n

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens int32 [T] on the device; returns fp32 logits of the last row [vocab]."""
        from .. import ops
        c, go = self.cfg, self.go
        T = tokens.numel()
        if self.pos + T > self.max_context:
            raise ValueError("context exceeds max_context")
        pos = torch.arange(self.pos, self.pos + T, device=self.device, dtype=torch.int32)
        logits = self._forward_at(tokens, pos)
        self.pos += T
        return logits

    @torch.no_grad()
    def _forward_at(self, tokens: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """The forward pass with the positions given as a device tensor (nothing here depends on host-side position
        arithmetic, so a single-token call can be captured into a CUDA graph)."""
        from .. import ops
        c, go = self.cfg, self.go
        T = tokens.numel()
        h = go.gguf_dequant_rows(self.embed, self.types["token_embd.weight"], c.dim, tokens)
        for i, L in enumerate(self.layers):
            b = f"blk.{i}."
            ta = self.types[b + "attn_q.weight"]
            nq, nkv = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
            if "qkv" in L:                                       # one projection for q, k and v (same block type): rows q | k | v
                qkv = go.gguf_linear(h, L["qkv"], ta, nq + 2 * nkv, gamma=L["attn_norm"], eps=c.norm_eps)
                q, k, v = qkv[:, :nq], qkv[:, nq:nq + nkv], qkv[:, nq + nkv:]
            else:
                q = go.gguf_linear(h, L["q"], ta, nq, gamma=L["attn_norm"], eps=c.norm_eps)
                k = go.gguf_linear(h, L["k"], self.types[b + "attn_k.weight"], nkv, gamma=L["attn_norm"], eps=c.norm_eps)
                v = go.gguf_linear(h, L["v"], self.types[b + "attn_v.weight"], nkv, gamma=L["attn_norm"], eps=c.norm_eps)
            # whole-vector RMS with per-element gamma, rotation at `pos`, k / v appended to the caches: one kernel
            q = ops.full_qk_norm_rope_append(q, k, v, pos, L["q_norm"], L["k_norm"], self.rope_cos, self.rope_sin, L["kc"], L["vc"],
                                             n_heads=c.n_heads, n_kv_heads=c.n_kv_heads, rope_dim=c.rope_dim, eps=c.norm_eps)
            # prefill chunks (consecutive positions) through the tcgen05 flash kernel, decode steps through the split kernel
            o = ops.gqa_prefill(q, L["kc"], L["vc"], pos) if T >= 16 else ops.gqa_decode(q, L["kc"], L["vc"], pos, nsplit=1 if T > 8 else 8)
            att = go.gguf_linear(o, L["o"], self.types[b + "attn_output.weight"], c.dim, epi=2)
            h = (h + att).to(torch.bfloat16)                     # bf16 + fp32 promotes to fp32: the sum is rounded once
            xn = ops.rmsnorm(h, L["ffn_norm"], mode=2, eps=c.norm_eps)
            ids, wt = go.router_topk(xn, L["router"], c.n_experts_used, bias=L["bias"], score_func="sigmoid", norm_topk=True)
            if self.balanced_routes:
                # benchmark aid for random weights (whose hidden states collapse and send every token to the same few
                # experts): the router still runs, but token t uses experts (t * k + j + 37 * layer) mod E with equal weights
                kk = c.n_experts_used
                ids = ((pos.view(-1, 1) * kk + torch.arange(kk, device=self.device, dtype=torch.int32).view(1, -1) + 37 * i) % c.n_experts).to(torch.int32).contiguous()
                wt = torch.full_like(wt, 1.0 / kk)
            if "cache" in L:
                from ..moe.expert_cache import staged_moe_forward
                # routes to other ranks' experts become weight-0 routes to this rank's first expert: they add exactly nothing
                mine = (ids >= self.e_start) & (ids < self.e_start + self.e_local)
                y = staged_moe_forward(L["cache"], xn, torch.where(mine, ids - self.e_start, torch.zeros_like(ids)).contiguous(),
                                       torch.where(mine, wt, torch.zeros_like(wt)).contiguous(), self.types[b + "ffn_gate_exps.weight"],
                                       self.types[b + "ffn_down_exps.weight"], c.expert_inter)
                if self.world > 1:
                    self._combine(y)
                h = (h + y).to(torch.bfloat16)
                continue
            routes = go.group_routes(ids, wt, c.n_experts)
            # many routes per expert (prefill): grouped tensor-core GEMMs; else the per-route streaming kernels
            y = go.moe_forward(xn, L["w13"], L["w2"], self.types[b + "ffn_gate_exps.weight"], self.types[b + "ffn_down_exps.weight"],
                               c.n_experts, c.expert_inter, routes, expert_offset=self.e_start, local_experts=self.e_local, peer=self._peer())
            if self.world > 1 and not routes.combined:
                self._combine(y)
            h = (h + y).to(torch.bfloat16)
        return go.gguf_linear(h[-1:], self.head, self.types["output.weight"], c.vocab_size, gamma=self.final_norm, eps=c.norm_eps, epi=2)[0]

    def forward_logits(self, tokens: Sequence[int]) -> torch.Tensor:
        """fp32 logits after feeding `tokens` at the current position (for host-side sampling and log-probabilities)."""
        return self.forward(torch.tensor(list(tokens), dtype=torch.int32, device=self.device))

    # protocol of the generic generation runtime
    def _checked(self, token: int) -> int:
        """The step's token, or `StepFailed` on every rank when a peer all-reduce timed out (collective check; the
        token was read from the device just before, so the step is complete)."""
        if self._combiner is not None:
            self._combiner.check_step(self.device)
        return token

    def prefill(self, tokens: Sequence[int]) -> int:
        t = torch.tensor(list(tokens), dtype=torch.int32, device=self.device)
        return self._checked(int(torch.argmax(self.forward(t))))

    @torch.no_grad()
    def _capture_decode(self) -> None:
        self._tok_buf = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._pos_buf = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._next_buf = torch.zeros((), dtype=torch.int64, device=self.device)
        self._pos_buf.fill_(self.pos)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):                       # warm-up outside the capture: lazy kernel attributes, allocator
            self._forward_at(self._tok_buf, self._pos_buf)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._next_buf.copy_(torch.argmax(self._forward_at(self._tok_buf, self._pos_buf)))
        self._graph = g

    def decode_one(self, token: int) -> int:
        if not self.use_graph:
            return self._checked(int(torch.argmax(self.forward(torch.tensor([token], dtype=torch.int32, device=self.device)))))
        if self.pos + 1 > self.max_context:
            raise ValueError("context exceeds max_context")
        if self._graph is None:
            self._capture_decode()
        self._tok_buf.fill_(int(token))
        self._pos_buf.fill_(self.pos)
        self._graph.replay()
        self.pos += 1
        nxt = int(self._next_buf)
        try:
            return self._checked(nxt)
        except TimeoutError:
            self._graph = None     # the captured graph holds the peer all-reduce; recapture on the NCCL path
            raise
