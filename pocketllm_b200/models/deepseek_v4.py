"""DeepSeek-V4 family: configuration, random checkpoints, and a stateless fp32 oracle.

Architecture (reference: src/models/deepseek_v4/runtime.py - ModelArgs 501-575, Compressor
1011-1109, Indexer 1112-1288, Attention 1291-1659, Gate 1662-1731, Block 4256-4476,
ParallelHead 4479-4586, MTPBlock 4589-4621):

* The residual stream is `hc_mult` (4) parallel copies. Before each sub-layer `hc_pre` mixes them
  into one vector with sigmoid weights and produces `post` (4) and a Sinkhorn-normalised `comb`
  (4x4); after it `hc_post` writes `h'_j = post_j * y + sum_i comb[i][j] * h_i`.
* Attention is multi-query with ONE shared 512-wide key/value vector per token (K == V):
  low-rank q (`wq_a` -> RMSNorm -> `wq_b`), per-head RMS scaling without gamma, RoPE on the last 64
  dims (interleaved pairs), FP8 fake quantisation (blocks of 64, power-of-two scales) of the 448
  non-rotary KV dims. A query sees the last `window_size` tokens plus *compressed* entries: every
  `ratio` tokens a softmax-gated pooling of per-token (kv, score) projections emits one entry
  (ratio 4 pools over two overlapping blocks). Ratio-4 layers pick the `index_topk` best entries
  with a lightning indexer (64 heads x 128, Hadamard-rotated, FP4 fake-quantised; score
  `sum_h w_h * relu(q_h . k_c)`); ratio-128 layers use every entry. The softmax has one extra
  per-head sink logit in the denominator. Output: inverse RoPE, grouped low-rank `wo_a`, `wo_b`.
* FFN: `sqrt(softplus)` router scores, bias only for selection, weights normalised and scaled by
  `route_scale`; the first `n_hash_layers` layers take expert ids from a `tid2eid[token]` table;
  SwiGLU experts with clamping (`swiglu_limit`), FP4 (E2M1 + E8M0 per 32) weights; one shared expert.
* Head: sigmoid-weighted mix of the copies, RMSNorm, vocabulary projection. MTP block: a full block
  fed with `e_proj(norm(embed(token))) + h_proj(norm(h))` plus its own head mix.

The oracle below is *stateless*: it defines every quantity as a function of the whole token prefix
(entry c of a ratio-r compressor covers tokens [c*r, (c+1)*r) and is visible to position p when
`(p+1)//r > c`). The GPU runtime (`deepseek_v4_runtime.py`) keeps rings and pooling state and must
agree with it position by position. Linear layers use weight-only quantisation here (activations
stay in higher precision than the reference's FP8 activation quantisation).
"""
from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch
import torch.nn.functional as F

from ..formats import fp4 as fp4fmt


@dataclass
class DSV4Config:
    vocab_size: int = 129280
    dim: int = 4096
    moe_inter_dim: int = 2048
    n_layers: int = 43
    n_hash_layers: int = 3
    n_mtp_layers: int = 1
    n_heads: int = 64
    n_routed_experts: int = 256
    n_shared_experts: int = 1
    n_activated_experts: int = 6
    score_func: str = "sqrtsoftplus"
    route_scale: float = 1.5
    swiglu_limit: float = 10.0
    q_lora_rank: int = 1024
    head_dim: int = 512
    rope_head_dim: int = 64
    norm_eps: float = 1e-6
    o_groups: int = 8
    o_lora_rank: int = 1024
    window_size: int = 128
    compress_ratios: tuple = (0, 0) + (4, 128) * 20 + (4, 0)     # n_layers + 1 (last entry: MTP block)
    compress_rope_theta: float = 160000.0
    original_seq_len: int = 65536
    rope_theta: float = 10000.0
    rope_factor: float = 16.0
    beta_fast: int = 32
    beta_slow: int = 1
    index_n_heads: int = 64
    index_head_dim: int = 128
    index_topk: int = 512
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    max_seq_len: int = 4096

    @classmethod
    def tiny(cls, **kw) -> "DSV4Config":
        """Every mechanism present (hash + scored routing, window-only / ratio-4 + indexer / ratio-128
        layers with a 16-token stand-in for 128, MTP) at unit-test size."""
        base = dict(vocab_size=512, dim=256, moe_inter_dim=256, n_layers=4, n_hash_layers=1, n_mtp_layers=1, n_heads=4,
                    n_routed_experts=8, n_activated_experts=2, q_lora_rank=256, head_dim=128, rope_head_dim=64, o_groups=2,
                    o_lora_rank=128, window_size=16, compress_ratios=(0, 4, 16, 4, 0), original_seq_len=64, rope_factor=4.0,
                    index_n_heads=4, index_head_dim=128, index_topk=6, max_seq_len=256)
        base.update(kw)
        return cls(**base)

    @classmethod
    def from_json(cls, text_or_path: str | Path) -> "DSV4Config":
        text = str(text_or_path)
        d = json.loads(text if text.lstrip().startswith("{") else Path(text).read_text())
        known = {k: v for k, v in d.items() if k in cls.__dataclass_fields__}
        if "compress_ratios" in known:
            known["compress_ratios"] = tuple(known["compress_ratios"])
        return cls(**known)

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    def ratio(self, layer: int) -> int:
        return int(self.compress_ratios[layer]) if layer < len(self.compress_ratios) else 0

    @property
    def mix_hc(self) -> int:
        return (2 + self.hc_mult) * self.hc_mult


# ---------------------------------------------------------------------------------------
# numerics shared by the oracle and the runtime's CPU fallbacks

_FP4_LEVELS = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def pow2_ceil(x: torch.Tensor) -> torch.Tensor:
    return torch.pow(2.0, torch.ceil(torch.log2(x.clamp_min(torch.finfo(torch.float32).tiny))))


def fp8_fake_quant(x: torch.Tensor, block: int = 64) -> torch.Tensor:
    """Per-`block` E4M3 round trip with a power-of-two scale (amax clamped at 1e-4)."""
    shp = x.shape
    v = x.float().reshape(-1, shp[-1] // block, block)
    s = pow2_ceil(v.abs().amax(-1, keepdim=True).clamp_min(1e-4) / 448.0)
    q = (v / s).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
    return (q * s).reshape(shp)


def fp4_fake_quant(x: torch.Tensor, block: int = 32) -> torch.Tensor:
    """Per-`block` E2M1 round trip (nearest level, first level on ties) with a power-of-two scale."""
    shp = x.shape
    v = x.float().reshape(-1, shp[-1] // block, block)
    s = pow2_ceil(v.abs().amax(-1, keepdim=True).clamp_min(6.0 * 2.0 ** -126) / 6.0)
    n = (v / s).clamp(-6.0, 6.0)
    lv = _FP4_LEVELS.to(x.device)
    q = lv[(n.unsqueeze(-1) - lv).abs().argmin(-1)]
    return (q * s).reshape(shp)


def hadamard128(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard transform of the last dim (128, Sylvester order)."""
    v = x.float()
    n = v.shape[-1]
    h = 1
    while h < n:
        v = v.reshape(*v.shape[:-1], n // (2 * h), 2, h)
        v = torch.stack([v[..., 0, :] + v[..., 1, :], v[..., 0, :] - v[..., 1, :]], dim=-2)
        v = v.reshape(*v.shape[:-3], n)
        h *= 2
    return v * (n ** -0.5)


def rmsnorm(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    x = x.float()
    y = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.float()


def rope_angles(cfg: DSV4Config, compressed_layer: bool, positions: torch.Tensor) -> torch.Tensor:
    """[len(positions), rope_head_dim/2] angles. Layers with compression use `compress_rope_theta`
    with YaRN interpolation; pure window layers use `rope_theta` without it."""
    rd = cfg.rope_head_dim
    base = cfg.compress_rope_theta if compressed_layer else cfg.rope_theta
    freqs = 1.0 / (base ** (torch.arange(0, rd, 2, dtype=torch.float64) / rd))
    if compressed_layer and cfg.original_seq_len > 0:
        def corr(rot):
            return rd * math.log(cfg.original_seq_len / (rot * 2 * math.pi)) / (2 * math.log(base))
        low, high = max(math.floor(corr(cfg.beta_fast)), 0), min(math.ceil(corr(cfg.beta_slow)), rd - 1)
        if low == high:
            high += 0.001
        smooth = 1 - ((torch.arange(rd // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        freqs = freqs / cfg.rope_factor * (1 - smooth) + freqs * smooth
    return torch.outer(positions.double().cpu(), freqs)


def apply_rope(x: torch.Tensor, ang: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate interleaved pairs (x[2i], x[2i+1]) of the last dim by `ang` [..., rd/2] (broadcast)."""
    c, s = torch.cos(ang).float().to(x.device), torch.sin(ang).float().to(x.device)
    if inverse:
        s = -s
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack([a * c - b * s, a * s + b * c], dim=-1).flatten(-2)


def hc_split(mix: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, hc: int, iters: int, eps: float):
    """mix [..., (2+hc)*hc] -> pre [..., hc], post [..., hc], comb [..., hc, hc]."""
    pre = torch.sigmoid(mix[..., :hc] * scale[0] + base[:hc]) + eps
    post = 2 * torch.sigmoid(mix[..., hc:2 * hc] * scale[1] + base[hc:2 * hc])
    comb = (mix[..., 2 * hc:] * scale[2] + base[2 * hc:]).reshape(*mix.shape[:-1], hc, hc)
    comb = torch.softmax(comb, -1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(max(iters - 1, 0)):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return pre, post, comb


def hc_pre(h: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, cfg: DSV4Config):
    """h [T, hc, dim] -> x [T, dim], post [T, hc], comb [T, hc, hc]."""
    flat = h.float().flatten(1)
    mix = (flat @ fn.float().T) * torch.rsqrt(flat.square().mean(-1, keepdim=True) + cfg.norm_eps)
    pre, post, comb = hc_split(mix, scale.float(), base.float(), cfg.hc_mult, cfg.hc_sinkhorn_iters, cfg.hc_eps)
    return (pre.unsqueeze(-1) * h.float()).sum(1), post, comb


def hc_post(y: torch.Tensor, h: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    return post.unsqueeze(-1) * y.float().unsqueeze(1) + torch.einsum("tij,tid->tjd", comb, h.float())


def hc_head(h: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, cfg: DSV4Config) -> torch.Tensor:
    flat = h.float().flatten(1)
    mix = (flat @ fn.float().T) * torch.rsqrt(flat.square().mean(-1, keepdim=True) + cfg.norm_eps)
    pre = torch.sigmoid(mix * scale.float() + base.float()) + cfg.hc_eps
    return (pre.unsqueeze(-1) * h.float()).sum(1)


def route(x: torch.Tensor, gate_w: torch.Tensor, bias: torch.Tensor | None, tid2eid: torch.Tensor | None, tokens: torch.Tensor,
          cfg: DSV4Config, forced_idx: torch.Tensor | None = None):
    s = x.float() @ gate_w.float().T
    s = s.softmax(-1) if cfg.score_func == "softmax" else s.sigmoid() if cfg.score_func == "sigmoid" else F.softplus(s).sqrt()
    if forced_idx is not None:
        idx = forced_idx.long()
    elif tid2eid is not None:
        idx = tid2eid[tokens].long()
    else:
        idx = (s + bias.float() if bias is not None else s).topk(cfg.n_activated_experts, -1)[1]
    w = s.gather(1, idx)
    if cfg.score_func != "softmax":
        w = w / w.sum(-1, keepdim=True)
    return w * cfg.route_scale, idx


def swiglu(gate: torch.Tensor, up: torch.Tensor, limit: float) -> torch.Tensor:
    if limit > 0:
        up = up.clamp(-limit, limit)
        gate = gate.clamp(max=limit)
    return F.silu(gate) * up


# ---------------------------------------------------------------------------------------
# checkpoints

def _linear_names(prefix: str, ratio: int) -> list[str]:
    n = [f"{prefix}.attn.{k}" for k in ("wq_a", "wq_b", "wkv", "wo_a", "wo_b")]
    return n


def random_checkpoint(cfg: DSV4Config, seed: int = 0, sigma: float = 0.05) -> dict[str, torch.Tensor]:
    """Random weights under the reference's tensor names. Dense weights are bf16-representable fp32;
    routed experts are stored as FP4 (`.weight` uint8 nibbles + `.scale` E8M0 per 32)."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=sigma):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).float()

    W: dict[str, torch.Tensor] = {}
    d, hd, H = cfg.dim, cfg.head_dim, cfg.n_heads
    W["embed.weight"] = rnd(cfg.vocab_size, d, s=1.0)
    W["norm.weight"] = 1 + rnd(d, s=0.1)
    W["head.weight"] = rnd(cfg.vocab_size, d)
    W["hc_head_fn"], W["hc_head_base"], W["hc_head_scale"] = rnd(cfg.hc_mult, cfg.hc_mult * d), rnd(cfg.hc_mult, s=0.5), 1 + rnd(1, s=0.1)

    def block(p: str, layer: int):
        ratio = cfg.ratio(layer)
        for kind in ("attn", "ffn"):
            W[f"{p}.hc_{kind}_fn"] = rnd(cfg.mix_hc, cfg.hc_mult * d)
            W[f"{p}.hc_{kind}_base"] = rnd(cfg.mix_hc, s=0.5)
            W[f"{p}.hc_{kind}_scale"] = 1 + rnd(3, s=0.1)
        W[f"{p}.attn_norm.weight"], W[f"{p}.ffn_norm.weight"] = 1 + rnd(d, s=0.1), 1 + rnd(d, s=0.1)
        a = f"{p}.attn"
        W[f"{a}.wq_a.weight"], W[f"{a}.q_norm.weight"] = rnd(cfg.q_lora_rank, d), 1 + rnd(cfg.q_lora_rank, s=0.1)
        W[f"{a}.wq_b.weight"] = rnd(H * hd, cfg.q_lora_rank)
        W[f"{a}.wkv.weight"], W[f"{a}.kv_norm.weight"] = rnd(hd, d), 1 + rnd(hd, s=0.1)
        W[f"{a}.attn_sink"] = rnd(H, s=1.0)
        W[f"{a}.wo_a.weight"] = rnd(cfg.o_groups * cfg.o_lora_rank, H * hd // cfg.o_groups)
        W[f"{a}.wo_b.weight"] = rnd(d, cfg.o_groups * cfg.o_lora_rank)

        def compressor(c: str, r: int, cd: int):
            coff = 2 if r == 4 else 1
            W[f"{c}.ape"] = rnd(r, coff * cd, s=0.5)
            W[f"{c}.wkv.weight"], W[f"{c}.wgate.weight"] = rnd(coff * cd, d), rnd(coff * cd, d, s=4 * sigma)
            W[f"{c}.norm.weight"] = 1 + rnd(cd, s=0.1)
        if ratio:
            compressor(f"{a}.compressor", ratio, hd)
            if ratio == 4:
                W[f"{a}.indexer.wq_b.weight"] = rnd(cfg.index_n_heads * cfg.index_head_dim, cfg.q_lora_rank)
                W[f"{a}.indexer.weights_proj.weight"] = rnd(cfg.index_n_heads, d, s=4 * sigma)
                compressor(f"{a}.indexer.compressor", ratio, cfg.index_head_dim)
        f = f"{p}.ffn"
        W[f"{f}.gate.weight"] = rnd(cfg.n_routed_experts, d, s=4 * sigma)
        if layer < cfg.n_hash_layers:
            W[f"{f}.gate.tid2eid"] = torch.stack([torch.randperm(cfg.n_routed_experts, generator=g)[:cfg.n_activated_experts]
                                                  for _ in range(cfg.vocab_size)]).to(torch.int32)
        else:
            W[f"{f}.gate.bias"] = rnd(cfg.n_routed_experts, s=0.2)
        for e in range(cfg.n_routed_experts):
            for name, (n, k) in (("w1", (cfg.moe_inter_dim, d)), ("w3", (cfg.moe_inter_dim, d)), ("w2", (d, cfg.moe_inter_dim))):
                packed, scale = fp4fmt.quantize_e2m1(torch.randn(n, k, generator=g) * sigma)
                W[f"{f}.experts.{e}.{name}.weight"], W[f"{f}.experts.{e}.{name}.scale"] = packed, scale
        si = cfg.n_shared_experts * cfg.moe_inter_dim
        W[f"{f}.shared_experts.w1.weight"], W[f"{f}.shared_experts.w3.weight"] = rnd(si, d), rnd(si, d)
        W[f"{f}.shared_experts.w2.weight"] = rnd(d, si)

    for i in range(cfg.n_layers):
        block(f"layers.{i}", i)
    for m in range(cfg.n_mtp_layers):
        p = f"mtp.{m}"
        block(p, cfg.n_layers + m)
        W[f"{p}.e_proj.weight"], W[f"{p}.h_proj.weight"] = rnd(d, d), rnd(d, d)
        for n in ("enorm", "hnorm", "norm"):
            W[f"{p}.{n}.weight"] = 1 + rnd(d, s=0.1)
        W[f"{p}.hc_head_fn"], W[f"{p}.hc_head_base"], W[f"{p}.hc_head_scale"] = rnd(cfg.hc_mult, cfg.hc_mult * d), rnd(cfg.hc_mult, s=0.5), 1 + rnd(1, s=0.1)
    return W


def expert_weight(W: dict, name: str) -> torch.Tensor:
    """fp32 matrix of a routed expert (`name` without the `.weight` suffix): FP4 nibbles + E8M0 scales, or already dense."""
    w = W[name + ".weight"]
    if w.is_floating_point():
        return w.float()
    return fp4fmt.dequantize_e2m1(w, W[name + ".scale"])


# ---------------------------------------------------------------------------------------
# oracle

class DSV4Oracle:
    """Whole-prefix fp32 evaluation on any device. `forward(tokens)` -> (logits [T, vocab], hidden
    [T, hc, dim]); `mtp_logits(hidden, next_tokens)` evaluates the MTP block."""

    def __init__(self, cfg: DSV4Config, weights: dict[str, torch.Tensor], device: str = "cpu"):
        self.cfg, self.dev = cfg, device
        # Discrete choices can be pinned to compare another implementation given the same choices:
        # force["<block>.ffn.route_idx"] = [T, k] expert ids, force["<block>.attn.index_sel"] = per position a
        # list of compressed-entry ids (or None for "all visible").
        self.force: dict = {}
        self.W = {k: v.to(device) for k, v in weights.items()}
        self._experts: dict[str, torch.Tensor] = {}
        self.trace: dict[str, torch.Tensor] = {}

    def _expert(self, name: str) -> torch.Tensor:
        if name not in self._experts:
            self._experts[name] = expert_weight(self.W, name).to(self.dev)
        return self._experts[name]

    # -- compressed entries -----------------------------------------------------------
    def _compress(self, xn: torch.Tensor, p: str, ratio: int, cd: int, rotate: bool, pos0: int = 0) -> torch.Tensor:
        """All complete entries of the prefix: [T // ratio, cd]."""
        W, cfg = self.W, self.cfg
        T = xn.shape[0]
        n = T // ratio
        if n == 0:
            return xn.new_zeros(0, cd)
        kv = xn @ W[f"{p}.wkv.weight"].T
        sc = xn @ W[f"{p}.wgate.weight"].T + W[f"{p}.ape"][torch.arange(T, device=xn.device) % ratio]
        kv, sc = kv[: n * ratio].reshape(n, ratio, -1), sc[: n * ratio].reshape(n, ratio, -1)
        if ratio == 4:                                    # overlapping pooling over the previous and the current block
            prev_kv = torch.cat([kv.new_zeros(1, ratio, cd), kv[:-1, :, :cd]], 0)
            prev_sc = torch.cat([sc.new_full((1, ratio, cd), float("-inf")), sc[:-1, :, :cd]], 0)
            kv, sc = torch.cat([prev_kv, kv[:, :, cd:]], 1), torch.cat([prev_sc, sc[:, :, cd:]], 1)
        ent = (kv * sc.softmax(1)).sum(1)
        ent = rmsnorm(ent, W[f"{p}.norm.weight"], cfg.norm_eps)
        rd = cfg.rope_head_dim
        ang = rope_angles(cfg, True, torch.arange(n) * ratio + pos0)
        ent = torch.cat([ent[:, :-rd], apply_rope(ent[:, -rd:], ang)], -1)
        if rotate:
            return fp4_fake_quant(hadamard128(ent))
        return torch.cat([fp8_fake_quant(ent[:, :-rd]), ent[:, -rd:]], -1)

    # -- attention ---------------------------------------------------------------------
    def _attention(self, xn: torch.Tensor, p: str, layer: int) -> torch.Tensor:
        W, cfg = self.W, self.cfg
        T, H, hd, rd = xn.shape[0], cfg.n_heads, cfg.head_dim, cfg.rope_head_dim
        ratio = cfg.ratio(layer)
        pos = torch.arange(T)
        ang = rope_angles(cfg, ratio != 0, pos)
        qr = rmsnorm(xn @ W[f"{p}.wq_a.weight"].T, W[f"{p}.q_norm.weight"], cfg.norm_eps)
        q = rmsnorm((qr @ W[f"{p}.wq_b.weight"].T).view(T, H, hd), None, cfg.norm_eps)
        q = torch.cat([q[..., :-rd], apply_rope(q[..., -rd:], ang.unsqueeze(1))], -1)
        kv = rmsnorm(xn @ W[f"{p}.wkv.weight"].T, W[f"{p}.kv_norm.weight"], cfg.norm_eps)
        kv = torch.cat([fp8_fake_quant(kv[:, :-rd]), apply_rope(kv[:, -rd:], ang)], -1)
        comp = self._compress(xn, f"{p}.compressor", ratio, hd, False) if ratio else None
        self.trace[f"{p}.q"], self.trace[f"{p}.kv"], self.trace[f"{p}.comp"] = q, kv, comp
        sel = None
        if ratio == 4:
            ih, idim = cfg.index_n_heads, cfg.index_head_dim
            iq = (qr @ W[f"{p}.indexer.wq_b.weight"].T).view(T, ih, idim)
            iq = torch.cat([iq[..., :-rd], apply_rope(iq[..., -rd:], ang.unsqueeze(1))], -1)
            iq = fp4_fake_quant(hadamard128(iq))
            ik = self._compress(xn, f"{p}.indexer.compressor", ratio, idim, True)
            w = (xn @ W[f"{p}.indexer.weights_proj.weight"].T) * (idim ** -0.5 * ih ** -0.5)
            score = (torch.einsum("thd,cd->thc", iq, ik).relu() * w.unsqueeze(-1)).sum(1)       # [T, n_entries]
            self.trace[f"{p}.index_score"], self.trace[f"{p}.index_k"] = score, ik
            sel = score
        scale = hd ** -0.5
        sink = W[f"{p}.attn_sink"].float()
        out = xn.new_zeros(T, H, hd)
        for t in range(T):
            rows = [kv[max(0, t - cfg.window_size + 1): t + 1]]
            if ratio:
                nvalid = (t + 1) // ratio
                if nvalid:
                    forced = self.force.get(f"{p}.index_sel")
                    if forced is not None and forced[t] is not None:
                        rows.append(comp[torch.as_tensor(forced[t], device=comp.device, dtype=torch.long)])
                    elif sel is not None and nvalid > cfg.index_topk:
                        keep = sel[t, :nvalid].topk(cfg.index_topk)[1]
                        rows.append(comp[keep])
                    else:
                        rows.append(comp[:nvalid])
            k = torch.cat(rows, 0)
            s = torch.einsum("hd,nd->hn", q[t], k) * scale
            pr = torch.softmax(torch.cat([s, sink.unsqueeze(1)], 1), -1)[:, :-1]
            out[t] = pr @ k
        out = torch.cat([out[..., :-rd], apply_rope(out[..., -rd:], ang.unsqueeze(1), inverse=True)], -1)
        self.trace[f"{p}.o"] = out
        G = cfg.o_groups
        og = out.reshape(T, G, H // G * hd)
        wo_a = W[f"{p}.wo_a.weight"].view(G, cfg.o_lora_rank, -1)
        o = torch.einsum("tgd,grd->tgr", og, wo_a).reshape(T, -1)
        return o @ W[f"{p}.wo_b.weight"].T

    # -- FFN ---------------------------------------------------------------------------
    def _ffn(self, xn: torch.Tensor, p: str, layer: int, tokens: torch.Tensor) -> torch.Tensor:
        W, cfg = self.W, self.cfg
        forced = self.force.get(f"{p}.route_idx")
        w, idx = route(xn, W[f"{p}.gate.weight"], W.get(f"{p}.gate.bias"), W.get(f"{p}.gate.tid2eid"), tokens, cfg,
                       None if forced is None else forced.to(xn.device))
        self.trace[f"{p}.route_idx"], self.trace[f"{p}.route_w"] = idx, w
        y = torch.zeros_like(xn)
        for e in idx.unique().tolist():
            tsel, ksel = (idx == e).nonzero(as_tuple=True)
            xe = xn[tsel]
            h = swiglu(xe @ self._expert(f"{p}.experts.{e}.w1").T, xe @ self._expert(f"{p}.experts.{e}.w3").T, cfg.swiglu_limit)
            y.index_add_(0, tsel, (h * w[tsel, ksel].unsqueeze(-1)) @ self._expert(f"{p}.experts.{e}.w2").T)
        s = f"{p}.shared_experts"
        h = swiglu(xn @ W[f"{s}.w1.weight"].T, xn @ W[f"{s}.w3.weight"].T, cfg.swiglu_limit)
        return y + h @ W[f"{s}.w2.weight"].T

    def _block(self, h: torch.Tensor, p: str, layer: int, tokens: torch.Tensor) -> torch.Tensor:
        W, cfg = self.W, self.cfg
        x, post, comb = hc_pre(h, W[f"{p}.hc_attn_fn"], W[f"{p}.hc_attn_scale"], W[f"{p}.hc_attn_base"], cfg)
        y = self._attention(rmsnorm(x, W[f"{p}.attn_norm.weight"], cfg.norm_eps), f"{p}.attn", layer)
        h = hc_post(y, h, post, comb)
        x, post, comb = hc_pre(h, W[f"{p}.hc_ffn_fn"], W[f"{p}.hc_ffn_scale"], W[f"{p}.hc_ffn_base"], cfg)
        y = self._ffn(rmsnorm(x, W[f"{p}.ffn_norm.weight"], cfg.norm_eps), f"{p}.ffn", layer, tokens)
        return hc_post(y, h, post, comb)

    @torch.no_grad()
    def forward(self, tokens) -> tuple[torch.Tensor, torch.Tensor]:
        W, cfg = self.W, self.cfg
        tokens = torch.as_tensor(tokens, device=self.dev).long()
        h = W["embed.weight"][tokens].float().unsqueeze(1).repeat(1, cfg.hc_mult, 1)
        for i in range(cfg.n_layers):
            h = self._block(h, f"layers.{i}", i, tokens)
            self.trace[f"layers.{i}.out"] = h
        x = hc_head(h, W["hc_head_fn"], W["hc_head_scale"], W["hc_head_base"], cfg)
        return rmsnorm(x, W["norm.weight"], cfg.norm_eps) @ W["head.weight"].float().T, h

    @torch.no_grad()
    def mtp_logits(self, hidden: torch.Tensor, next_tokens, m: int = 0) -> torch.Tensor:
        """MTP block `m` over the whole prefix: position t combines the backbone hidden of position t
        with the embedding of token t+1 (`next_tokens[t]`) and predicts token t+2."""
        W, cfg = self.W, self.cfg
        p = f"mtp.{m}"
        nt = torch.as_tensor(next_tokens, device=self.dev).long()
        e = rmsnorm(W["embed.weight"][nt], W[f"{p}.enorm.weight"], cfg.norm_eps)
        x = rmsnorm(hidden, W[f"{p}.hnorm.weight"], cfg.norm_eps)
        h = (e @ W[f"{p}.e_proj.weight"].T).unsqueeze(1) + x @ W[f"{p}.h_proj.weight"].T
        h = self._block(h, p, cfg.n_layers + m, nt)
        x = hc_head(h, W[f"{p}.hc_head_fn"], W[f"{p}.hc_head_scale"], W[f"{p}.hc_head_base"], cfg)
        return rmsnorm(x, W[f"{p}.norm.weight"], cfg.norm_eps) @ W["head.weight"].float().T

    def greedy(self, prompt, n: int) -> list[int]:
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(self.forward(toks)[0][-1].argmax()))
        return toks[len(prompt):]
