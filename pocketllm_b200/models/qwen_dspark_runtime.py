"""GPU runtime of the external DSpark block drafter of the Qwen hybrid model, on the framework's kernels: tcgen05 bf16 GEMMs
for every projection, the fused q / k RMSNorm + YaRN rotation + cache append kernel, split-context GQA attention over
context + block, and the Markov head kernels (`csrc/kernels/dspark.cu`); plus the speculative loop that couples it to the
native engine through target taps, verify rows and snapshots.

Definition and fp32 oracle: `qwen_dspark.py`. Reference: cpp_engine/src/qwen_dspark.cpp:598-640 (append_target_taps),
686-829 (propose), 874- (speculative generate), cpp_engine/cuda/qwen_dspark_ops.cu.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int

import torch

from .. import ops
from ..ops import _check, _ptr, _stream
from ..ops import lib as _lib
from .qwen_dspark import QwenDSparkConfig, yarn_inv_freq


class QwenDSparkRuntime:
    """`append_target_taps(taps, position)` commits context rows, `propose(anchor)` drafts a block, `crop_context(position)`
    forgets a rejected suffix. Weights are the drafter checkpoint's tensors (bf16), `embed` / `lm_head` the target's."""

    def __init__(self, cfg: QwenDSparkConfig, weights: dict[str, torch.Tensor], embed: torch.Tensor, lm_head: torch.Tensor, *, max_context: int = 4096,
                 device: str | torch.device = "cuda"):
        if cfg.head_dim != 128:
            raise ValueError("the drafter kernels take head_dim 128")
        self.cfg, self.device, self.max_context = cfg, torch.device(device), max_context
        dev = self.device
        bf = lambda t: t.to(dev, torch.bfloat16).contiguous()
        f32 = lambda t: t.to(dev, torch.float32).contiguous()
        W = weights
        self.fc, self.hidden_norm, self.norm = bf(W["fc.weight"]), f32(W["hidden_norm.weight"]), f32(W["norm.weight"])
        self.w1, self.w2 = bf(W["markov_head.markov_w1.weight"]), bf(W["markov_head.markov_w2.weight"])
        self.conf_w, self.conf_b = f32(W["confidence_head.proj.weight"]).view(-1), f32(W["confidence_head.proj.bias"])
        self.embed, self.lm_head = bf(embed), bf(lm_head)
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            self.layers.append({
                "in_ln": f32(W[p + "input_layernorm.weight"]), "post_ln": f32(W[p + "post_attention_layernorm.weight"]),
                "qkv": bf(torch.cat([W[p + "self_attn.q_proj.weight"], W[p + "self_attn.k_proj.weight"], W[p + "self_attn.v_proj.weight"]], 0)),
                "kv": bf(torch.cat([W[p + "self_attn.k_proj.weight"], W[p + "self_attn.v_proj.weight"]], 0)),
                "o": bf(W[p + "self_attn.o_proj.weight"]), "q_norm": f32(W[p + "self_attn.q_norm.weight"]), "k_norm": f32(W[p + "self_attn.k_norm.weight"]),
                "gate_up": bf(torch.cat([W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"]], 0)), "down": bf(W[p + "mlp.down_proj.weight"]),
                "kc": torch.zeros(cfg.num_key_value_heads, max_context, 128, device=dev, dtype=torch.bfloat16),
                "vc": torch.zeros(cfg.num_key_value_heads, max_context, 128, device=dev, dtype=torch.bfloat16)})
        ang = torch.outer(torch.arange(max_context, dtype=torch.float64), yarn_inv_freq(cfg))
        self.cos_t = (torch.cos(ang) * cfg.attention_factor()).float().to(dev).contiguous()
        self.sin_t = (torch.sin(ang) * cfg.attention_factor()).float().to(dev).contiguous()
        self.nq, self.nkv = cfg.num_attention_heads * 128, cfg.num_key_value_heads * 128
        self._cand_v = torch.empty(592, device=dev, dtype=torch.float32)
        self._cand_i = torch.empty(592, device=dev, dtype=torch.int32)
        self.committed = 0

    def reset(self) -> None:
        self.committed = 0

    def crop_context(self, position: int) -> None:
        """Forget committed rows at and after `position` (the caches are position indexed: nothing is copied)."""
        self.committed = min(self.committed, position)

    def _qk(self, q, k, v, pos, L, n_q_heads: int) -> torch.Tensor | None:
        c = self.cfg
        M = k.shape[0]
        q_out = torch.empty(M, n_q_heads, 128, device=self.device, dtype=torch.bfloat16) if n_q_heads else None
        st = _lib.kernels().pk_dspark_qk_norm_rope_append(
            _ptr(q), c_int(0 if q is None else q.stride(0)), _ptr(k), c_int(k.stride(0)), _ptr(v), c_int(v.stride(0)), _ptr(pos), c_int(M), c_int(n_q_heads),
            c_int(c.num_key_value_heads), c_int(128), _ptr(L["q_norm"]), _ptr(L["k_norm"]), _ptr(self.cos_t), _ptr(self.sin_t), c_float(c.rms_norm_eps),
            _ptr(q_out), _ptr(L["kc"]), _ptr(L["vc"]), c_int(self.max_context), _stream())
        _check(st, "pk_dspark_qk_norm_rope_append")
        return q_out

    @torch.no_grad()
    def append_target_taps(self, taps: torch.Tensor, position: int) -> None:
        """taps bf16 [rows, n_taps * hidden] of target positions position .. position + rows - 1 (in order, no gaps)."""
        if position != self.committed:
            raise ValueError("target taps must be appended in position order without gaps")
        rows = taps.shape[0]
        if position + rows + self.cfg.block_size > self.max_context:
            raise ValueError("drafter context exceeds max_context")
        ctx = ops.rmsnorm(ops.gemm_bf16(taps.contiguous(), self.fc), self.hidden_norm, mode=2, eps=self.cfg.rms_norm_eps)
        pos = torch.arange(position, position + rows, device=self.device, dtype=torch.int32)
        for L in self.layers:
            kv = ops.gemm_bf16(ctx, L["kv"])
            self._qk(None, kv[:, : self.nkv], kv[:, self.nkv:], pos, L, 0)
        self.committed += rows

    @torch.no_grad()
    def propose(self, anchor: int | torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(draft tokens int32 [block] on the device, confidences fp32 [block], Markov-corrected logits fp32 [block, vocab]).
        `anchor` may be a device tensor: nothing here waits for the host."""
        c = self.cfg
        B, dev = c.block_size, self.device
        anchor_t = anchor.to(dev, torch.int32).view(1) if isinstance(anchor, torch.Tensor) else torch.tensor([anchor], device=dev, dtype=torch.int32)
        ids = torch.cat([anchor_t, torch.full((B - 1,), c.mask_token_id, device=dev, dtype=torch.int32)])
        h = self.embed.index_select(0, ids.long())
        pos = torch.arange(self.committed, self.committed + B, device=dev, dtype=torch.int32)
        extent = torch.full((B,), self.committed + B - 1, device=dev, dtype=torch.int32)      # every row sees the context and the whole block
        for L in self.layers:
            x = ops.rmsnorm(h, L["in_ln"], mode=2, eps=c.rms_norm_eps)
            qkv = ops.gemm_bf16(x, L["qkv"])
            q = self._qk(qkv[:, : self.nq], qkv[:, self.nq:self.nq + self.nkv], qkv[:, self.nq + self.nkv:], pos, L, c.num_attention_heads)
            att = ops.gqa_decode(q, L["kc"], L["vc"], extent, nsplit=8)
            h = ops.gemm_bf16(att, L["o"], epi=ops.EPI_RESID, resid=h)
            x = ops.rmsnorm(h, L["post_ln"], mode=2, eps=c.rms_norm_eps)
            h = ops.gemm_bf16(ops.gemm_bf16(x, L["gate_up"], epi=ops.EPI_SWIGLU), L["down"], epi=ops.EPI_RESID, resid=h)
        hn = ops.rmsnorm(h, self.norm, mode=2, eps=c.rms_norm_eps)
        logits = ops.gemm_bf16(hn, self.lm_head, epi=ops.EPI_F32)
        K = _lib.kernels()
        e = torch.empty(c.markov_rank, device=dev, dtype=torch.float32)
        emb = torch.empty(B, c.markov_rank, device=dev, dtype=torch.float32)
        tokens = torch.empty(B, device=dev, dtype=torch.int32)
        _check(K.pk_dspark_markov_embed(_ptr(anchor_t), _ptr(self.w1), c_int(c.markov_rank), _ptr(e), _stream()), "pk_dspark_markov_embed")
        for r in range(B):
            emb[r].copy_(e)
            _check(K.pk_dspark_markov_row(_ptr(logits[r]), _ptr(self.w2), _ptr(self.w1), _ptr(e), c_int(c.vocab_size), c_int(c.markov_rank), _ptr(self._cand_v),
                                          _ptr(self._cand_i), c_int(592), _ptr(tokens[r:]), _ptr(e), _stream()), "pk_dspark_markov_row")
        conf = torch.sigmoid(torch.cat([hn.float(), emb], -1) @ self.conf_w + self.conf_b)
        return tokens, conf, logits


class QwenDSparkSpeculator:
    """Greedy speculative generation: the drafter proposes a block after every committed token, the engine verifies up to
    seven drafts at once (`forward_rows`), rewinds to its snapshot and replays the accepted prefix when a draft is wrong, and
    hands the drafter the taps of the rows it kept. The tokens equal the engine's plain greedy decode."""

    def __init__(self, engine, drafter: QwenDSparkRuntime, max_draft: int | None = None, min_confidence: float = 0.0):
        self.eng, self.d = engine, drafter
        self.max_draft = min(max_draft or drafter.cfg.block_size, drafter.cfg.block_size, 7)
        self.min_confidence = min_confidence
        engine.set_tap_layers(list(drafter.cfg.target_layer_ids))
        self.stats = {"rounds": 0, "proposed": 0, "accepted": 0, "rollbacks": 0}

    def prefill(self, prompt, chunk: int = 512) -> int:
        self.d.reset()
        first, pos = -1, 0
        chunk = max(1, min(chunk, int(getattr(self.eng, "prefill_chunk", chunk) or chunk)))     # the taps hold one engine chunk
        for lo in range(0, len(prompt), chunk):
            piece = list(prompt[lo:lo + chunk])
            first = self.eng.prefill(piece)
            self.d.append_target_taps(self.eng.taps(), pos)
            pos += len(piece)
        return first

    def generate(self, prompt, max_new_tokens: int, chunk: int = 512) -> list[int]:
        self.eng.reset()
        first = self.prefill(prompt, chunk)
        return ([first] + self.decode(first, max_new_tokens - 1))[:max_new_tokens]

    def decode(self, first: int, n: int) -> list[int]:
        """`n` tokens after `first` (the token the prefill produced, not yet consumed by the target)."""
        eng, d = self.eng, self.d
        max_new_tokens = n + 1
        out = [first]
        snap = eng.snapshot()
        try:
            while len(out) < max_new_tokens:
                anchor = out[-1]
                committed = eng.position
                toks, conf, _ = d.propose(anchor)
                k = min(self.max_draft, max_new_tokens - len(out) - 1)
                drafts, confs = toks[:k].tolist(), conf[:k].tolist()
                for i, cf in enumerate(confs):              # stop the block at the first draft the confidence head doubts
                    if cf < self.min_confidence:
                        drafts = drafts[:i]
                        break
                rows = [anchor] + drafts
                snap.update()
                preds = eng.forward_rows(rows)
                correct = 0
                while correct < len(drafts) and preds[correct] == drafts[correct]:
                    correct += 1
                self.stats["rounds"] += 1
                self.stats["proposed"] += len(drafts)
                if correct < len(drafts):
                    # rows behind the first wrong draft advanced the recurrent state: rewind and replay what is kept
                    while True:
                        self.stats["rollbacks"] += 1
                        snap.restore()
                        preds = eng.forward_rows(rows[:correct + 1])
                        agree = 0
                        while agree < correct and preds[agree] == drafts[agree]:
                            agree += 1
                        if agree == correct:
                            break
                        correct = agree
                self.stats["accepted"] += correct
                d.append_target_taps(eng.taps(0, correct + 1), committed)
                out += drafts[:correct] + [preds[correct]]
        finally:
            snap.free()
        return out[1:max_new_tokens]
