"""External DSpark block drafter for the Qwen hybrid model: configuration, the 62-tensor checkpoint layout, a random
checkpoint writer and the fp32 definition of `append_target_taps` / `propose`. The native engine does not run this
drafter yet (it drafts with the checkpoint's own multi-token predictor); this module fixes the numerics the native
version has to reproduce and serves as its oracle.

Structure (reference: cpp_engine/src/qwen_dspark.cpp:348-419 tensors, 598-640 context append, 686-829 proposal):

* taps: the target's hidden states after layers `target_layer_ids` (default 4, 16, 28, 40, 52), concatenated ->
  `fc` [hidden, n_taps * hidden] -> RMSNorm (`hidden_norm`, plain gamma) = the context row of a committed position.
* every drafter layer (standard attention + SwiGLU MLP, per-head q / k RMSNorm, YaRN rotation on the whole head) keeps
  a context K/V cache filled from those rows; a proposal runs `block_size` rows [anchor token, mask, mask, ...] at
  positions committed .. committed + block_size - 1, each row attending to the whole context and to ALL rows of the
  block (no causal mask inside the block).
* head: `norm`, the target's lm_head, then row by row the Markov bias `w2 @ w1[previous token]` and a greedy pick, and
  a confidence `sigmoid(w . [hidden, w1[previous]] + b)` per row.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class QwenDSparkConfig:
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 5
    num_attention_heads: int = 40
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 151936
    block_size: int = 7
    markov_rank: int = 256
    mask_token_id: int = 151935
    target_layer_ids: tuple = (4, 16, 28, 40, 52)
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1.0e6
    rope_factor: float = 1.0                 # YaRN: 1 = plain rotation
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    rope_original_max_positions: int = 32768
    rope_attention_factor: float | None = None

    def attention_factor(self) -> float:
        if self.rope_attention_factor is not None:
            return self.rope_attention_factor
        return 0.1 * math.log(self.rope_factor) + 1.0 if self.rope_factor > 1.0 else 1.0

    def validate_for_target(self, hidden: int, vocab: int, layers: int) -> None:
        if self.hidden_size != hidden or self.vocab_size != vocab:
            raise ValueError("drafter hidden size / vocabulary do not match the target model")
        if not self.target_layer_ids or max(self.target_layer_ids) >= layers or min(self.target_layer_ids) < 0:
            raise ValueError("target_layer_ids must name layers of the target model")
        if not 0 <= self.mask_token_id < self.vocab_size or self.head_dim % 2 or self.block_size < 1:
            raise ValueError("mask token, head_dim or block size out of range")

    @classmethod
    def tiny(cls, hidden: int = 128, vocab: int = 512, target_layers: int = 4) -> "QwenDSparkConfig":
        return cls(hidden_size=hidden, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                   vocab_size=vocab, block_size=4, markov_rank=16, mask_token_id=vocab - 1, target_layer_ids=(1, target_layers - 1),
                   rope_theta=10000.0)


def tensor_names(cfg: QwenDSparkConfig) -> list[tuple[str, tuple[int, ...]]]:
    """Every tensor of a drafter checkpoint with its shape (7 + 11 per layer; 62 for the published 5-layer drafter)."""
    H, I, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    q, kv, T = cfg.num_attention_heads * D, cfg.num_key_value_heads * D, len(cfg.target_layer_ids)
    out = [("fc.weight", (H, H * T)), ("hidden_norm.weight", (H,)), ("norm.weight", (H,)),
           ("markov_head.markov_w1.weight", (cfg.vocab_size, cfg.markov_rank)), ("markov_head.markov_w2.weight", (cfg.vocab_size, cfg.markov_rank)),
           ("confidence_head.proj.weight", (1, H + cfg.markov_rank)), ("confidence_head.proj.bias", (1,))]
    for i in range(cfg.num_hidden_layers):
        p = f"layers.{i}."
        out += [(p + "input_layernorm.weight", (H,)), (p + "post_attention_layernorm.weight", (H,)),
                (p + "self_attn.q_proj.weight", (q, H)), (p + "self_attn.k_proj.weight", (kv, H)), (p + "self_attn.v_proj.weight", (kv, H)),
                (p + "self_attn.o_proj.weight", (H, q)), (p + "self_attn.q_norm.weight", (D,)), (p + "self_attn.k_norm.weight", (D,)),
                (p + "mlp.gate_proj.weight", (I, H)), (p + "mlp.up_proj.weight", (I, H)), (p + "mlp.down_proj.weight", (H, I))]
    return out


def random_checkpoint(cfg: QwenDSparkConfig, seed: int = 0, sigma: float = 0.05) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_names(cfg):
        if name.endswith("norm.weight"):
            t = 1.0 + 0.05 * torch.randn(*shape, generator=g)
        elif name.endswith(".bias"):
            t = 0.1 * torch.randn(*shape, generator=g)
        else:
            t = sigma * torch.randn(*shape, generator=g) * (4.0 if "markov" in name else 1.0)
        out[name] = t.to(torch.bfloat16)
    return out


def save_checkpoint(directory, cfg: QwenDSparkConfig, weights: dict[str, torch.Tensor]) -> None:
    """A drafter directory: `config.json` (the dataclass fields) and the tensors of `tensor_names` as Safetensors."""
    import dataclasses
    import json
    from pathlib import Path
    from ..formats import safetensors_io as st_io
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    fields = dataclasses.asdict(cfg)
    fields["target_layer_ids"] = list(cfg.target_layer_ids)
    (d / "config.json").write_text(json.dumps(fields, indent=1))
    st_io.write_sharded(d, {k: v.contiguous() for k, v in weights.items()})


def load_checkpoint(directory) -> tuple[QwenDSparkConfig, dict[str, torch.Tensor]]:
    """(config, tensors) of a drafter directory; every tensor of `tensor_names` must be present with its shape."""
    import json
    from pathlib import Path
    from ..formats import safetensors_io as st_io
    d = Path(directory)
    fields = json.loads((d / "config.json").read_text())
    known = {f for f in QwenDSparkConfig.__dataclass_fields__}
    cfg = QwenDSparkConfig(**{k: (tuple(v) if k == "target_layer_ids" else v) for k, v in fields.items() if k in known})
    model = st_io.SafetensorsModel(d)
    tensors = {k: model.get(k).clone() for k in model.keys()}
    for name, shape in tensor_names(cfg):
        if name not in tensors:
            raise ValueError(f"drafter checkpoint lacks {name}")
        if tuple(tensors[name].shape) != tuple(shape):
            raise ValueError(f"{name}: shape {tuple(tensors[name].shape)} where {tuple(shape)} is expected")
    return cfg, tensors


def yarn_inv_freq(cfg: QwenDSparkConfig) -> torch.Tensor:
    """Inverse frequencies of the rotation [head_dim / 2] (fp64): plain for factor 1, else the YaRN blend of
    interpolated and extrapolated frequencies between the beta_fast / beta_slow correction dims."""
    D = cfg.head_dim
    base = torch.pow(torch.tensor(cfg.rope_theta, dtype=torch.float64), -torch.arange(0, D, 2, dtype=torch.float64) / D)
    if cfg.rope_factor <= 1.0:
        return base

    def corr(rot: float) -> float:
        return D * math.log(cfg.rope_original_max_positions / (rot * 2 * math.pi)) / (2 * math.log(cfg.rope_theta))

    lo, hi = max(math.floor(corr(cfg.rope_beta_fast)), 0), min(math.ceil(corr(cfg.rope_beta_slow)), D // 2 - 1)
    ramp = ((torch.arange(D // 2, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
    return base / cfg.rope_factor * ramp + base * (1 - ramp)


class QwenDSparkOracle:
    """fp32 definition. `append_target_taps(taps, position)` commits rows; `propose(anchor)` drafts a block."""

    def __init__(self, cfg: QwenDSparkConfig, weights: dict[str, torch.Tensor], embed: torch.Tensor, lm_head: torch.Tensor):
        self.cfg = cfg
        self.W = {k: v.float() for k, v in weights.items()}
        self.embed, self.lm_head = embed.float(), lm_head.float()
        self.inv_freq = yarn_inv_freq(cfg)
        self.reset()

    def reset(self) -> None:
        self.committed = 0
        self.ctx_k = [[] for _ in range(self.cfg.num_hidden_layers)]      # per layer: list of [kv_heads, D] rows
        self.ctx_v = [[] for _ in range(self.cfg.num_hidden_layers)]

    def _norm(self, x: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + self.cfg.rms_norm_eps) * g

    def _rope(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """x [rows, heads, D]; half-split rotation over the whole head, scaled by the YaRN attention factor."""
        ang = positions.double()[:, None] * self.inv_freq[None, :]
        cs, sn = (torch.cos(ang) * self.cfg.attention_factor()).float()[:, None, :], (torch.sin(ang) * self.cfg.attention_factor()).float()[:, None, :]
        half = self.cfg.head_dim // 2
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn], -1)

    def _kv(self, layer: int, x: torch.Tensor, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        c, p = self.cfg, f"layers.{layer}.self_attn."
        k = (x @ self.W[p + "k_proj.weight"].T).view(-1, c.num_key_value_heads, c.head_dim)
        v = (x @ self.W[p + "v_proj.weight"].T).view(-1, c.num_key_value_heads, c.head_dim)
        return self._rope(self._norm(k, self.W[p + "k_norm.weight"]), positions), v

    @torch.no_grad()
    def append_target_taps(self, taps: torch.Tensor, position: int) -> None:
        """taps [rows, n_taps * hidden] of the target positions position .. position + rows - 1 (in order, no gaps)."""
        if position != self.committed:
            raise ValueError("target taps must be appended in position order without gaps")
        ctx = self._norm(taps.float() @ self.W["fc.weight"].T, self.W["hidden_norm.weight"])
        pos = torch.arange(position, position + taps.shape[0])
        for l in range(self.cfg.num_hidden_layers):
            k, v = self._kv(l, ctx, pos)
            self.ctx_k[l] += list(k)
            self.ctx_v[l] += list(v)
        self.committed += taps.shape[0]

    def crop_context(self, position: int) -> None:
        """Forget committed rows at and after `position` (a rejected verify suffix)."""
        for l in range(self.cfg.num_hidden_layers):
            del self.ctx_k[l][position:]
            del self.ctx_v[l][position:]
        self.committed = min(self.committed, position)

    @torch.no_grad()
    def propose(self, anchor: int) -> tuple[list[int], torch.Tensor, torch.Tensor]:
        """(draft tokens [block_size], confidences [block_size], Markov-corrected logits [block_size, vocab])."""
        c, W = self.cfg, self.W
        B, Hq, Hkv, D = c.block_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim
        ids = torch.full((B,), c.mask_token_id, dtype=torch.long)
        ids[0] = anchor
        pos = torch.arange(self.committed, self.committed + B)
        h = self.embed[ids]
        for l in range(c.num_hidden_layers):
            p = f"layers.{l}."
            x = self._norm(h, W[p + "input_layernorm.weight"])
            q = self._rope(self._norm((x @ W[p + "self_attn.q_proj.weight"].T).view(B, Hq, D), W[p + "self_attn.q_norm.weight"]), pos)
            bk, bv = self._kv(l, x, pos)
            K = torch.stack(self.ctx_k[l] + list(bk)) if self.ctx_k[l] else bk        # [ctx + B, Hkv, D]: every row sees all of it
            V = torch.stack(self.ctx_v[l] + list(bv)) if self.ctx_v[l] else bv
            rep = Hq // Hkv
            s = torch.einsum("bhd,nhd->bhn", q, K.repeat_interleave(rep, 1)) * D ** -0.5
            o = torch.einsum("bhn,nhd->bhd", torch.softmax(s, -1), V.repeat_interleave(rep, 1)).reshape(B, Hq * D)
            h = h + o @ W[p + "self_attn.o_proj.weight"].T
            x = self._norm(h, W[p + "post_attention_layernorm.weight"])
            h = h + (torch.nn.functional.silu(x @ W[p + "mlp.gate_proj.weight"].T) * (x @ W[p + "mlp.up_proj.weight"].T)) @ W[p + "mlp.down_proj.weight"].T
        hn = self._norm(h, W["norm.weight"])
        logits = hn @ self.lm_head.T
        w1, w2 = W["markov_head.markov_w1.weight"], W["markov_head.markov_w2.weight"]
        tokens, emb, prev = [], [], anchor
        for r in range(B):
            e = w1[prev]
            logits[r] += w2 @ e
            emb.append(e)
            prev = int(logits[r].argmax())
            tokens.append(prev)
        conf = torch.sigmoid(torch.cat([hn, torch.stack(emb)], -1) @ W["confidence_head.proj.weight"].T + W["confidence_head.proj.bias"]).squeeze(-1)
        return tokens, conf, logits
