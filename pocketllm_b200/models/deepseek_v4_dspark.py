"""DSpark multi-token drafter for DeepSeek-V4: a few extra blocks under the `mtp.*` names that draft `block_size`
tokens from one committed token, reading their keys and values from the backbone's hidden states.

Structure (reference: src/models/deepseek_v4/dspark.py:40-275, loop src/models/deepseek_v4/dspark_loop.py:77-253):

* target taps: the outputs of `target_layer_ids` (mean over the hyper-connection copies), concatenated, go through
  `mtp.0.main_proj` and `mtp.0.main_norm` -> `main_x` [T, dim].
* every stage is a DSV4 block without compression whose attention takes K/V of the *committed* positions from `main_x`
  (own window ring) and K/V of the draft block from its own input; each draft query sees the whole committed window
  and all keys of the draft block.
* draft input: the committed token followed by `block_size - 1` noise tokens, at positions p+1 .. p+block_size.
* last stage: head mix + norm + vocabulary head, then a rank-`markov_rank` bigram bias applied position by position
  (`logits[i] += markov_w2 @ markov_w1[previous token]`), greedy pick, and a confidence score per draft token.

`DSparkOracle` is the fp32 definition; `DSparkDrafter` runs on the GPU kernels of the DSV4 runtime;
`generate_dspark` is the gated speculative loop (draft, truncate by the cost model, verify in one multi-row pass,
rewind by position).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from . import deepseek_v4 as d4


@dataclass
class DSparkConfig:
    n_stages: int = 3
    block_size: int = 5
    target_layer_ids: tuple = (40, 41, 42)
    markov_rank: int = 256
    noise_token_id: int = 0

    @classmethod
    def tiny(cls, cfg: d4.DSV4Config) -> "DSparkConfig":
        return cls(n_stages=2, block_size=4, target_layer_ids=(cfg.n_layers - 2, cfg.n_layers - 1), markov_rank=64, noise_token_id=1)


def stage_config(cfg: d4.DSV4Config, ds: DSparkConfig) -> d4.DSV4Config:
    """The backbone's config extended so that layer ids n_layers .. n_layers + n_stages - 1 are uncompressed, scored-routing blocks."""
    ratios = tuple(cfg.compress_ratios[: cfg.n_layers]) + (0,) * ds.n_stages
    return d4.DSV4Config(**{**cfg.__dict__, "compress_ratios": ratios, "n_mtp_layers": 0})


def random_weights(cfg: d4.DSV4Config, ds: DSparkConfig, seed: int = 1, sigma: float = 0.05) -> dict[str, torch.Tensor]:
    """Drafter weights under `mtp.<stage>.*` (block tensors as in the backbone; embedding and head are the backbone's)."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *shape, s=sigma: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).float()
    sc = stage_config(cfg, ds)
    # reuse the block generator of the checkpoint writer: build a throw-away model with n_stages "MTP" blocks
    tmp = d4.DSV4Config(**{**sc.__dict__, "n_layers": 0, "n_hash_layers": 0, "n_mtp_layers": ds.n_stages,
                           "compress_ratios": (0,) * ds.n_stages})
    base = d4.random_checkpoint(tmp, seed=seed + 100, sigma=sigma)
    W = {k: v for k, v in base.items() if k.startswith("mtp.") and ".e_proj" not in k and ".h_proj" not in k and ".enorm" not in k and ".hnorm" not in k}
    last = ds.n_stages - 1
    for s in range(ds.n_stages):
        for k in ("norm.weight", "hc_head_fn", "hc_head_base", "hc_head_scale"):
            if s != last:
                W.pop(f"mtp.{s}.{k}", None)
    d = cfg.dim
    W["mtp.0.main_proj.weight"] = rnd(d, d * len(ds.target_layer_ids))
    W["mtp.0.main_norm.weight"] = 1 + rnd(d, s=0.1)
    W[f"mtp.{last}.markov_head.markov_w1.weight"] = rnd(cfg.vocab_size, ds.markov_rank, s=0.5)
    W[f"mtp.{last}.markov_head.markov_w2.weight"] = rnd(cfg.vocab_size, ds.markov_rank, s=0.5)
    W[f"mtp.{last}.confidence_head.proj.weight"] = rnd(1, d + ds.markov_rank, s=0.5)
    return W


def markov_decode(logits: torch.Tensor, committed: int, w1: torch.Tensor, w2: torch.Tensor) -> tuple[list[int], torch.Tensor, torch.Tensor]:
    """Position-by-position greedy pick with the bigram bias: (draft ids [B], biased logits [B, V], markov embeds [B, R])."""
    out, embeds, prev = [], [], committed
    logits = logits.clone()
    for i in range(logits.shape[0]):
        e = w1[prev].float()
        logits[i] += w2.float() @ e
        embeds.append(e)
        prev = int(logits[i].argmax())
        out.append(prev)
    return out, logits, torch.stack(embeds)


class DSparkOracle:
    """fp32 definition over a whole prefix: `draft(main_taps, tokens, p)` drafts from the token committed after position p,
    given the backbone's target taps for positions 0..p."""

    def __init__(self, cfg: d4.DSV4Config, ds: DSparkConfig, backbone: dict[str, torch.Tensor], weights: dict[str, torch.Tensor], device="cpu"):
        self.cfg, self.ds, self.dev = stage_config(cfg, ds), ds, device
        self.W = {k: v.to(device) for k, v in {**backbone, **weights}.items() if k.startswith(("mtp.", "embed.", "head."))}
        self.block = d4.DSV4Oracle(self.cfg, self.W, device)          # for its FFN and expert cache

    def main_x(self, taps: torch.Tensor) -> torch.Tensor:
        W = self.W
        return d4.rmsnorm(taps.float() @ W["mtp.0.main_proj.weight"].T, W["mtp.0.main_norm.weight"], self.cfg.norm_eps)

    def _attention(self, p: str, xn: torch.Tensor, main_x: torch.Tensor, pos_commit: int) -> torch.Tensor:
        """xn [B, dim] normalised draft inputs at positions pos_commit+1..; main_x [pos_commit+1, dim]."""
        W, cfg = self.W, self.cfg
        B, H, hd, rd = xn.shape[0], cfg.n_heads, cfg.head_dim, cfg.rope_head_dim
        def kv_of(x, positions):
            kv = d4.rmsnorm(x @ W[f"{p}.wkv.weight"].T, W[f"{p}.kv_norm.weight"], cfg.norm_eps)
            ang = d4.rope_angles(cfg, False, positions)
            return torch.cat([d4.fp8_fake_quant(kv[:, :-rd]), d4.apply_rope(kv[:, -rd:], ang)], -1)
        lo = max(0, pos_commit - cfg.window_size + 1)
        k_commit = kv_of(main_x[lo: pos_commit + 1], torch.arange(lo, pos_commit + 1))
        dpos = torch.arange(pos_commit + 1, pos_commit + 1 + B)
        k_draft = kv_of(xn, dpos)
        ang = d4.rope_angles(cfg, False, dpos)
        qr = d4.rmsnorm(xn @ W[f"{p}.wq_a.weight"].T, W[f"{p}.q_norm.weight"], cfg.norm_eps)
        q = d4.rmsnorm((qr @ W[f"{p}.wq_b.weight"].T).view(B, H, hd), None, cfg.norm_eps)
        q = torch.cat([q[..., :-rd], d4.apply_rope(q[..., -rd:], ang.unsqueeze(1))], -1)
        k = torch.cat([k_commit, k_draft], 0)
        s = torch.einsum("bhd,nd->bhn", q, k) * hd ** -0.5
        sink = W[f"{p}.attn_sink"].float().view(1, H, 1).expand(B, H, 1)
        pr = torch.softmax(torch.cat([s, sink], -1), -1)[..., :-1]
        o = torch.einsum("bhn,nd->bhd", pr, k)
        o = torch.cat([o[..., :-rd], d4.apply_rope(o[..., -rd:], ang.unsqueeze(1), inverse=True)], -1)
        G = cfg.o_groups
        o = torch.einsum("tgd,grd->tgr", o.reshape(B, G, H // G * hd), W[f"{p}.wo_a.weight"].view(G, cfg.o_lora_rank, -1)).reshape(B, -1)
        return o @ W[f"{p}.wo_b.weight"].T

    @torch.no_grad()
    def draft(self, taps: torch.Tensor, committed: int, pos_commit: int) -> tuple[list[int], torch.Tensor, torch.Tensor]:
        """taps [pos_commit + 1, n_targets * dim] -> (draft ids [B], confidence [B], biased logits [B, V])."""
        W, cfg, ds = self.W, self.cfg, self.ds
        main_x = self.main_x(taps.to(self.dev))
        ids = torch.full((ds.block_size,), ds.noise_token_id, dtype=torch.long, device=self.dev)
        ids[0] = committed
        h = W["embed.weight"][ids].float().unsqueeze(1).repeat(1, cfg.hc_mult, 1)
        for s in range(ds.n_stages):
            p = f"mtp.{s}"
            x, post, comb = d4.hc_pre(h, W[f"{p}.hc_attn_fn"], W[f"{p}.hc_attn_scale"], W[f"{p}.hc_attn_base"], cfg)
            y = self._attention(f"{p}.attn", d4.rmsnorm(x, W[f"{p}.attn_norm.weight"], cfg.norm_eps), main_x, pos_commit)
            h = d4.hc_post(y, h, post, comb)
            x, post, comb = d4.hc_pre(h, W[f"{p}.hc_ffn_fn"], W[f"{p}.hc_ffn_scale"], W[f"{p}.hc_ffn_base"], cfg)
            y = self.block._ffn(d4.rmsnorm(x, W[f"{p}.ffn_norm.weight"], cfg.norm_eps), f"{p}.ffn", cfg.n_layers + s, ids)
            h = d4.hc_post(y, h, post, comb)
        p = f"mtp.{ds.n_stages - 1}"
        x = d4.hc_head(h, W[f"{p}.hc_head_fn"], W[f"{p}.hc_head_scale"], W[f"{p}.hc_head_base"], cfg)
        logits = d4.rmsnorm(x, W[f"{p}.norm.weight"], cfg.norm_eps) @ W["head.weight"].float().T
        out, biased, emb = markov_decode(logits, committed, W[f"{p}.markov_head.markov_w1.weight"], W[f"{p}.markov_head.markov_w2.weight"])
        conf = (torch.cat([x.float(), emb], -1) @ W[f"{p}.confidence_head.proj.weight"].float().T).squeeze(-1)
        return out, conf, biased


class DSparkDrafter:
    """The drafter on the GPU, sharing the kernels, embedding and head of a `DSV4Runtime`."""

    def __init__(self, rt, ds: DSparkConfig, weights: dict[str, torch.Tensor]):
        from .deepseek_v4_runtime import _BlockState, _BlockWeights, _Lin
        self.rt, self.ds = rt, ds
        self.cfg = stage_config(rt.cfg, ds)
        W = weights
        f32 = lambda n: W[n].float().cuda().contiguous()
        self.stages = [_BlockWeights(self.cfg, W, f"mtp.{s}", rt.cfg.n_layers + s) for s in range(ds.n_stages)]
        self.state = [_BlockState(self.cfg, 0, rt.max_context, max(rt.max_rows, ds.block_size)) for _ in self.stages]
        # room for the draft block's own keys behind the ring
        for st in self.state:
            st.kv = torch.zeros(st.ring + ds.block_size, self.cfg.head_dim, device="cuda", dtype=torch.bfloat16)
        self.main_proj, self.main_norm = _Lin(W["mtp.0.main_proj.weight"]), f32("mtp.0.main_norm.weight")
        last = f"mtp.{ds.n_stages - 1}"
        self.norm = f32(f"{last}.norm.weight")
        self.hc_head = (f32(f"{last}.hc_head_fn"), f32(f"{last}.hc_head_scale"), f32(f"{last}.hc_head_base"))
        self.w1, self.w2 = f32(f"{last}.markov_head.markov_w1.weight"), f32(f"{last}.markov_head.markov_w2.weight")
        self.conf_w = f32(f"{last}.confidence_head.proj.weight")
        self.rows = torch.arange(ds.block_size, device="cuda", dtype=torch.int32)
        self.sel = self.rows.repeat(ds.block_size, 1).contiguous()

    def _main_x(self, taps: torch.Tensor) -> torch.Tensor:
        from .. import ops
        y = self.main_proj(taps.to(torch.bfloat16).contiguous(), f32=True)
        return ops.rmsnorm(y.to(torch.bfloat16).contiguous(), self.main_norm, mode=2, eps=self.cfg.norm_eps)

    @torch.no_grad()
    def write_main_kv(self, taps: torch.Tensor, pos0: int) -> None:
        """Committed positions pos0.. (taps [M, n_targets * dim]) enter every stage's window ring."""
        from ..ops import dsv4_ops as dk
        cfg = self.cfg
        cos_t, sin_t = self.rt.rope[False]
        mx = self._main_x(taps)
        for i in range(0, mx.shape[0], 8 * 64):
            part = mx[i: i + 8 * 64]
            pos_t = torch.arange(pos0 + i, pos0 + i + part.shape[0], device="cuda", dtype=torch.int32)
            for b, st in zip(self.stages, self.state):
                kv = b.proj(part, f32=True)[:, cfg.q_lora_rank: cfg.q_lora_rank + cfg.head_dim].contiguous()
                dk.kv_prep(kv, b.kv_norm, pos_t, cos_t, sin_t, cfg.rope_head_dim, st.ring, st.kv, cfg.norm_eps)

    @torch.no_grad()
    def draft(self, committed: int, pos_commit: int) -> tuple[list[int], torch.Tensor]:
        """Draft `block_size` tokens after `committed` (the token generated from position pos_commit, whose taps must have
        been written). Returns (draft ids, confidence [B] on the host)."""
        from .. import ops
        from ..ops import dsv4_ops as dk
        rt, cfg, ds = self.rt, self.cfg, self.ds
        B, H, hd, rd, ql = ds.block_size, cfg.n_heads, cfg.head_dim, cfg.rope_head_dim, cfg.q_lora_rank
        cos_t, sin_t = rt.rope[False]
        ids = torch.full((B,), ds.noise_token_id, device="cuda", dtype=torch.int32)
        ids[0] = committed
        dpos = torch.arange(pos_commit + 1, pos_commit + 1 + B, device="cuda", dtype=torch.int32)
        wpos = torch.full((B,), pos_commit, device="cuda", dtype=torch.int32)
        h = rt.embed[ids.long()].unsqueeze(1).repeat(1, cfg.hc_mult, 1).contiguous()
        kw = dict(iters=cfg.hc_sinkhorn_iters, hc_eps=cfg.hc_eps, norm_eps=cfg.norm_eps)
        for b, st in zip(self.stages, self.state):
            x, post, comb = dk.hc_pre(h, *b.hc_attn, b.attn_norm, **kw)
            A = b.proj(x, f32=True)
            qr = ops.rmsnorm(A[:, :ql].to(torch.bfloat16).contiguous(), b.q_norm, mode=2, eps=cfg.norm_eps)
            q = b.wq_b(qr).view(B, H, hd)
            dk.head_prep(q, dpos, cos_t, sin_t, rd, dk.PREP_NORM | dk.PREP_ROPE, cfg.norm_eps)
            # the draft block's keys go behind the ring: rows ring .. ring + B - 1 ("entries" 0 .. B-1 of the attention kernel)
            block_kv = st.kv[st.ring:]
            dk.kv_prep(A[:, ql:ql + hd].contiguous(), b.kv_norm, dpos, cos_t, sin_t, rd, st.ring, block_kv, cfg.norm_eps, dst_rows=self.rows)
            o = dk.sparse_attn(q, st.kv, wpos, b.sink, cos_t, sin_t, win=cfg.window_size, ring=st.ring, ratio=0, rd=rd, sel=self.sel, rope_pos=dpos)
            G = cfg.o_groups
            og = o.view(B, G, H // G * hd).transpose(0, 1).contiguous()
            y = b.wo_b(torch.cat([b.wo_a[g](og[g]) for g in range(G)], -1), f32=True)
            h = dk.hc_post(y, h, post, comb)
            x, post, comb = dk.hc_pre(h, *b.hc_ffn, b.ffn_norm, **kw)
            y, y2 = rt._ffn(b, x, ids)
            h = dk.hc_post(y, h, post, comb, y2=y2)
        x, raw = dk.hc_pre(h, *self.hc_head, self.norm, iters=0, hc_eps=cfg.hc_eps, norm_eps=cfg.norm_eps, head=True, want_raw=True)
        logits = rt.head(x, f32=True)
        out, _, emb = markov_decode(logits, committed, self.w1, self.w2)
        conf = (torch.cat([raw, emb], -1) @ self.conf_w.T).squeeze(-1)
        return out, conf.cpu()


def generate_dspark(rt, drafter: DSparkDrafter, prompt: Sequence[int], n: int, gate=None) -> tuple[list[int], dict]:
    """Greedy generation with DSpark drafts verified by the backbone. Equal to plain greedy decoding token for token."""
    ds = drafter.ds
    rt.tap_layers = tuple(ds.target_layer_ids)
    prompt = list(prompt)
    out = [rt.prefill(prompt)]
    drafter.write_main_kv(rt.last_taps, 0)
    stats = {"rounds": 0, "drafted": 0, "accepted": 0, "plain_steps": 0}
    while len(out) < n:
        p = rt.pos - 1                                     # last position the backbone has consumed
        room = n - len(out)
        ids, conf = ([], None)
        if room > 1 and (gate is None or gate.should_draft()):
            ids, conf = drafter.draft(out[-1], p)
            keep = len(ids) if gate is None else gate.choose_draft_len(torch.sigmoid(conf).tolist())
            ids = ids[: min(keep, room - 1, rt.max_rows - 1)]
        if not ids:
            nxt = rt.forward_rows([out[-1]])[0]
            drafter.write_main_kv(rt.last_taps, p + 1)
            out.append(nxt)
            stats["plain_steps"] += 1
            continue
        pred = rt.forward_rows([out[-1]] + ids)
        a = 0
        while a < len(ids) and pred[a] == ids[a]:
            a += 1
        stats["rounds"] += 1
        stats["drafted"] += len(ids)
        stats["accepted"] += a
        if gate is not None:
            gate.observe(torch.sigmoid(conf).tolist(), a, len(ids))
        rt.rollback(p + 2 + a)                             # rows 0..a stay: the committed token and the accepted drafts
        rt.last_token = pred[a]
        drafter.write_main_kv(rt.last_taps[: a + 1], p + 1)
        out += ids[:a] + [pred[a]]
    rt.tap_layers = ()
    return out[:n], stats
