"""Hybrid Gated-DeltaNet / GQA decoder (Qwen3.x-FP8 family).

* `QwenHybridConfig`      -- Hugging Face style config (same keys as the reference parses,
                             cpp_engine/src/qwen_config.cpp:105-151).
* `random_checkpoint`     -- random-init tensors in the on-disk FP8 layout with the reference's
                             tensor names (cpp_engine/src/qwen_weights.cpp:314-468).
* `ReferenceModel`        -- plain PyTorch fp32 restatement of the numerical contract
                             (cpp_engine/src/qwen_engine.cpp:960-1303, cuda/qwen_half_ops.cu:693-1158);
                             the oracle for kernel and engine tests.
* `QwenEngine`            -- the native engine (csrc/engine) behind a Python API: prefill,
                             CUDA-graph decode, speculative verify rows, snapshots.
"""
from __future__ import annotations

import ctypes
import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Sequence

import torch

from ..formats import fp8 as fp8fmt
from ..formats import safetensors_io as st_io
from ..ops import lib as _lib


@dataclass
class QwenHybridConfig:
    vocab_size: int = 151936
    hidden_size: int = 5120
    intermediate_size: int = 17408
    num_hidden_layers: int = 64
    num_attention_heads: int = 40
    num_key_value_heads: int = 8
    head_dim: int = 128
    attn_output_gate: bool = True
    rope_theta: float = 1.0e6
    partial_rotary_factor: float = 0.25
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 262144
    full_attention_interval: int = 4
    mtp_num_hidden_layers: int = 0
    layer_types: list[str] = field(default_factory=list)
    model_type: str = "qwen3_5_text"

    def __post_init__(self) -> None:
        if not self.layer_types:
            self.layer_types = ["full_attention" if (i + 1) % self.full_attention_interval == 0 else "linear_attention"
                                for i in range(self.num_hidden_layers)]

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor) & ~1

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @classmethod
    def from_json(cls, text: str) -> "QwenHybridConfig":
        d = json.loads(text)
        d = d.get("text_config", d)
        rp = d.get("rope_parameters") or {}
        names = {f for f in cls.__dataclass_fields__}
        kw = {k: v for k, v in d.items() if k in names}
        kw.update({k: v for k, v in rp.items() if k in names})
        return cls(**kw)

    @classmethod
    def benchmark_27b(cls) -> "QwenHybridConfig":
        """64 layers, hidden 5120, SwiGLU 17408, vocab 151936, 40/8 GQA heads, 16/32 DeltaNet heads."""
        return cls()

    @classmethod
    def tiny(cls, layers: int = 4, hidden: int = 256, inter: int = 512, vocab: int = 1024) -> "QwenHybridConfig":
        return cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                   num_attention_heads=4, num_key_value_heads=2, linear_num_key_heads=2, linear_num_value_heads=4,
                   max_position_embeddings=4096)


# --------------------------------------------------------------------------------------
# random checkpoints in the reference's tensor naming

def random_checkpoint(cfg: QwenHybridConfig, seed: int = 0, sigma: float = 0.02,
                      prefix: str = "model.language_model.", mtp: bool = False, mtp_bf16_linears: bool = False) -> dict[str, torch.Tensor]:
    """`mtp` adds the multi-token predictor (`mtp.*`: two input norms, fc, one full-attention layer, norm); its layer
    linears are FP8 like the backbone's, or plain bf16 with `mtp_bf16_linears`."""
    g = torch.Generator().manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    H, D = cfg.hidden_size, cfg.head_dim

    def fp8(name: str, n: int, k: int) -> None:
        w = torch.randn(n, k, generator=g) * sigma
        q, s = fp8fmt.quantize_block128(w)
        out[name + ".weight"] = q
        out[name + ".weight_scale_inv"] = s

    def bf16(name: str, *shape: int, mean: float = 0.0, std: float = sigma) -> None:
        out[name] = (mean + std * torch.randn(*shape, generator=g)).to(torch.bfloat16)

    bf16(prefix + "embed_tokens.weight", cfg.vocab_size, H)
    bf16(prefix + "norm.weight", H, std=0.05)
    bf16("lm_head.weight", cfg.vocab_size, H)
    KD = cfg.linear_num_key_heads * cfg.linear_key_head_dim
    VD = cfg.linear_num_value_heads * cfg.linear_value_head_dim
    for i, kind in enumerate(cfg.layer_types):
        p = f"{prefix}layers.{i}."
        bf16(p + "input_layernorm.weight", H, std=0.05)
        bf16(p + "post_attention_layernorm.weight", H, std=0.05)
        if kind == "linear_attention":
            fp8(p + "linear_attn.in_proj_qkv", 2 * KD + VD, H)
            fp8(p + "linear_attn.in_proj_z", VD, H)
            fp8(p + "linear_attn.out_proj", H, VD)
            bf16(p + "linear_attn.in_proj_a.weight", cfg.linear_num_value_heads, H)
            bf16(p + "linear_attn.in_proj_b.weight", cfg.linear_num_value_heads, H)
            bf16(p + "linear_attn.conv1d.weight", 2 * KD + VD, 1, cfg.linear_conv_kernel_dim, std=0.3)
            bf16(p + "linear_attn.A_log", cfg.linear_num_value_heads, std=0.5)
            bf16(p + "linear_attn.dt_bias", cfg.linear_num_value_heads, std=0.5)
            bf16(p + "linear_attn.norm.weight", cfg.linear_value_head_dim, mean=1.0, std=0.05)
        else:
            qd = cfg.num_attention_heads * D * (2 if cfg.attn_output_gate else 1)
            kvd = cfg.num_key_value_heads * D
            fp8(p + "self_attn.q_proj", qd, H)
            fp8(p + "self_attn.k_proj", kvd, H)
            fp8(p + "self_attn.v_proj", kvd, H)
            fp8(p + "self_attn.o_proj", H, cfg.num_attention_heads * D)
            bf16(p + "self_attn.q_norm.weight", D, std=0.05)
            bf16(p + "self_attn.k_norm.weight", D, std=0.05)
        fp8(p + "mlp.gate_proj", cfg.intermediate_size, H)
        fp8(p + "mlp.up_proj", cfg.intermediate_size, H)
        fp8(p + "mlp.down_proj", H, cfg.intermediate_size)
    if mtp:
        lin = (lambda name, n, k: bf16(name + ".weight", n, k)) if mtp_bf16_linears else fp8
        for name in ("pre_fc_norm_embedding", "pre_fc_norm_hidden", "norm"):
            bf16(f"mtp.{name}.weight", H, std=0.05)
        bf16("mtp.fc.weight", H, 2 * H)
        p = "mtp.layers.0."
        bf16(p + "input_layernorm.weight", H, std=0.05)
        bf16(p + "post_attention_layernorm.weight", H, std=0.05)
        lin(p + "self_attn.q_proj", cfg.num_attention_heads * D * (2 if cfg.attn_output_gate else 1), H)
        lin(p + "self_attn.k_proj", cfg.num_key_value_heads * D, H)
        lin(p + "self_attn.v_proj", cfg.num_key_value_heads * D, H)
        lin(p + "self_attn.o_proj", H, cfg.num_attention_heads * D)
        bf16(p + "self_attn.q_norm.weight", D, std=0.05)
        bf16(p + "self_attn.k_norm.weight", D, std=0.05)
        lin(p + "mlp.gate_proj", cfg.intermediate_size, H)
        lin(p + "mlp.up_proj", cfg.intermediate_size, H)
        lin(p + "mlp.down_proj", H, cfg.intermediate_size)
    return out


def save_checkpoint(directory: str | Path, cfg: QwenHybridConfig, tensors: dict[str, torch.Tensor],
                    max_shard_bytes: int = 4 << 30) -> None:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(cfg.to_json())
    st_io.write_sharded(d, tensors, max_shard_bytes=max_shard_bytes)


# --------------------------------------------------------------------------------------
# fp32 oracle

def _r16(x: torch.Tensor) -> torch.Tensor:
    """Round to bf16 and back: where the engine stores an activation in 16 bit."""
    return x.to(torch.bfloat16).float()


class ReferenceModel:
    """Token-by-token fp32 model with explicit state; small shapes only."""

    def __init__(self, cfg: QwenHybridConfig, tensors: dict[str, torch.Tensor], prefix: str = "model.language_model.",
                 emulate_bf16: bool = True, device: str = "cpu"):
        self.cfg, self.device = cfg, device
        self.r = _r16 if emulate_bf16 else (lambda x: x)
        self.p = prefix

        def lin(name: str) -> torch.Tensor:
            if name + ".weight_scale_inv" not in tensors:      # bf16 linear: the engine quantises it to FP8 blocks on load
                q, s = fp8fmt.quantize_block128(tensors[name + ".weight"].float(), scale_dtype=torch.float32)
                return fp8fmt.dequantize_block128(q, s).to(device)
            return fp8fmt.dequantize_block128(tensors[name + ".weight"], tensors[name + ".weight_scale_inv"]).to(device)

        def f(name: str) -> torch.Tensor:
            return tensors[name].float().to(device)

        self.embed, self.norm, self.lm_head = f(prefix + "embed_tokens.weight"), f(prefix + "norm.weight"), f("lm_head.weight")
        self.layers = []
        for i, kind in enumerate(cfg.layer_types):
            p = f"{prefix}layers.{i}."
            L = {"kind": kind, "in_norm": f(p + "input_layernorm.weight"), "post_norm": f(p + "post_attention_layernorm.weight"),
                 "gate": lin(p + "mlp.gate_proj"), "up": lin(p + "mlp.up_proj"), "down": lin(p + "mlp.down_proj")}
            if kind == "linear_attention":
                L.update(qkv=lin(p + "linear_attn.in_proj_qkv"), z=lin(p + "linear_attn.in_proj_z"), out=lin(p + "linear_attn.out_proj"),
                         a=f(p + "linear_attn.in_proj_a.weight"), b=f(p + "linear_attn.in_proj_b.weight"),
                         conv=f(p + "linear_attn.conv1d.weight").squeeze(1), A_log=f(p + "linear_attn.A_log"),
                         dt_bias=f(p + "linear_attn.dt_bias"), lnorm=f(p + "linear_attn.norm.weight"))
            else:
                L.update(q=lin(p + "self_attn.q_proj"), k=lin(p + "self_attn.k_proj"), v=lin(p + "self_attn.v_proj"),
                         o=lin(p + "self_attn.o_proj"), qn=f(p + "self_attn.q_norm.weight"), kn=f(p + "self_attn.k_norm.weight"))
            self.layers.append(L)
        self.mtp = None
        if "mtp.fc.weight" in tensors:
            p = "mtp.layers.0."
            self.mtp = {"kind": "full_attention", "in_norm": f(p + "input_layernorm.weight"), "post_norm": f(p + "post_attention_layernorm.weight"),
                        "gate": lin(p + "mlp.gate_proj"), "up": lin(p + "mlp.up_proj"), "down": lin(p + "mlp.down_proj"),
                        "q": lin(p + "self_attn.q_proj"), "k": lin(p + "self_attn.k_proj"), "v": lin(p + "self_attn.v_proj"),
                        "o": lin(p + "self_attn.o_proj"), "qn": f(p + "self_attn.q_norm.weight"), "kn": f(p + "self_attn.k_norm.weight"),
                        "norm_e": f("mtp.pre_fc_norm_embedding.weight"), "norm_h": f("mtp.pre_fc_norm_hidden.weight"),
                        "norm": f("mtp.norm.weight"), "fc": f("mtp.fc.weight")}
        self.reset()

    def reset(self) -> None:
        c = self.cfg
        KD = c.linear_num_key_heads * c.linear_key_head_dim
        VD = c.linear_num_value_heads * c.linear_value_head_dim
        self.pos = 0
        self.last_hidden = None          # the last step's hidden after the final norm (input of the predictor)
        self.mtp_kv = {}                 # position -> (k, v) of the predictor's layer
        self.state = []
        for L in self.layers:
            if L["kind"] == "linear_attention":
                self.state.append({"S": torch.zeros(c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim, device=self.device),
                                   "tail": torch.zeros(2 * KD + VD, c.linear_conv_kernel_dim - 1, device=self.device)})
            else:
                self.state.append({"k": [], "v": []})

    def _rms(self, x: torch.Tensor, g: torch.Tensor, plus_one: bool = True) -> torch.Tensor:
        r = torch.rsqrt((x * x).mean(-1, keepdim=True) + self.cfg.rms_norm_eps)
        return x * r * ((1.0 + g) if plus_one else g)

    def _linear_attn(self, L: dict, st: dict, x: torch.Tensor) -> torch.Tensor:
        c, r = self.cfg, self.r
        Hk, Hv, Dk, Dv = c.linear_num_key_heads, c.linear_num_value_heads, c.linear_key_head_dim, c.linear_value_head_dim
        KD, VD = Hk * Dk, Hv * Dv
        packed, z = r(L["qkv"] @ x), r(L["z"] @ x)
        a, b = r(L["a"] @ x), r(L["b"] @ x)
        window = torch.cat([st["tail"], packed[:, None]], dim=1)          # [C, 4]
        y = r(torch.nn.functional.silu((window * L["conv"]).sum(-1)))
        st["tail"] = window[:, 1:].clone()
        q, k, v = y[:KD].view(Hk, Dk), y[KD:2 * KD].view(Hk, Dk), y[2 * KD:].view(Hv, Dv)
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        rep = Hv // Hk
        q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)   # per value head
        g = -torch.exp(L["A_log"]) * torch.nn.functional.softplus(a + L["dt_bias"])
        beta = torch.sigmoid(b)
        S = st["S"] * torch.exp(g)[:, None, None]
        kv = torch.einsum("hkv,hk->hv", S, k)
        delta = (v - kv) * beta[:, None]
        S = S + torch.einsum("hk,hv->hkv", k, delta)
        st["S"] = S
        o = torch.einsum("hkv,hk->hv", S, q) * (Dk ** -0.5)
        o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + c.rms_norm_eps) * L["lnorm"] * torch.nn.functional.silu(z.view(Hv, Dv))
        return L["out"] @ r(o.reshape(VD))

    def _rope(self, x: torch.Tensor, pos: int) -> torch.Tensor:
        rd = self.cfg.rotary_dim
        if rd == 0:
            return x
        half = rd // 2
        inv = torch.pow(torch.tensor(self.cfg.rope_theta, dtype=torch.float64), -2.0 * torch.arange(half, dtype=torch.float64) / rd)
        ang = pos * inv
        cs, sn = torch.cos(ang).float().to(x.device), torch.sin(ang).float().to(x.device)
        x1, x2 = x[..., :half], x[..., half:rd]
        return torch.cat([x1 * cs - x2 * sn, x2 * cs + x1 * sn, x[..., rd:]], dim=-1)

    def _full_attn(self, L: dict, st: dict, x: torch.Tensor, pos: int) -> torch.Tensor:
        c, r = self.cfg, self.r
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        qg = r(L["q"] @ x).view(Hq, 2 * D) if c.attn_output_gate else None
        q = qg[:, :D] if qg is not None else r(L["q"] @ x).view(Hq, D)
        gate = qg[:, D:] if qg is not None else None
        k, v = r(L["k"] @ x).view(Hkv, D), r(L["v"] @ x).view(Hkv, D)
        q = r(self._rope(r(self._rms(q, L["qn"])), pos))
        k = r(self._rope(r(self._rms(k, L["kn"])), pos))
        st["k"].append(k)
        st["v"].append(v)
        K, V = torch.stack(st["k"], 1), torch.stack(st["v"], 1)          # [Hkv, T, D]
        rep = Hq // Hkv
        K, V = K.repeat_interleave(rep, 0), V.repeat_interleave(rep, 0)
        s = torch.einsum("hd,htd->ht", q, K) * (D ** -0.5)
        o = torch.einsum("ht,htd->hd", torch.softmax(s, -1), V)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return L["o"] @ r(o.reshape(Hq * D))

    def step(self, token: int) -> torch.Tensor:
        """Feed one token; returns fp32 logits [vocab]."""
        r = self.r
        h = self.embed[token].clone()
        layer_out = []
        for L, st in zip(self.layers, self.state):
            x = r(self._rms(h, L["in_norm"]))
            att = self._linear_attn(L, st, x) if L["kind"] == "linear_attention" else self._full_attn(L, st, x, self.pos)
            h = r(h + att)
            x = r(self._rms(h, L["post_norm"]))
            mid = r(torch.nn.functional.silu(L["gate"] @ x) * (L["up"] @ x))
            h = r(h + L["down"] @ mid)
            layer_out.append(h)
        self.layer_hidden = layer_out        # residual stream after every layer (the taps of an external drafter)
        self.pos += 1
        self.last_hidden = r(self._rms(h, self.norm))
        return self.lm_head @ self.last_hidden

    def mtp_step(self, token: int, hidden: torch.Tensor, pos: int) -> tuple[torch.Tensor, torch.Tensor]:
        """One predictor row: the token that FOLLOWS position `pos`, the (normalised) hidden of position `pos`; returns
        (logits for the token after that, the row's output after mtp.norm). Rows at later positions are forgotten first,
        as a position-indexed cache does. Reference: cpp_engine/src/qwen_engine.cpp:1423-1489."""
        r, L = self.r, self.mtp
        x = torch.cat([r(self._rms(self.embed[token], L["norm_e"])), r(self._rms(hidden, L["norm_h"]))])
        h = r(L["fc"] @ x)
        self.mtp_kv = {p: kv for p, kv in self.mtp_kv.items() if p < pos}
        order = sorted(self.mtp_kv)
        st = {"k": [self.mtp_kv[p][0] for p in order], "v": [self.mtp_kv[p][1] for p in order]}
        a = self._full_attn(L, st, r(self._rms(h, L["in_norm"])), pos)
        self.mtp_kv[pos] = (st["k"][-1], st["v"][-1])
        h = r(h + a)
        x = r(self._rms(h, L["post_norm"]))
        h = r(h + L["down"] @ r(torch.nn.functional.silu(L["gate"] @ x) * (L["up"] @ x)))
        out = r(self._rms(h, L["norm"]))
        return self.lm_head @ out, out

    def generate(self, prompt: Sequence[int], max_new_tokens: int) -> tuple[list[int], list[torch.Tensor]]:
        logits = None
        for t in prompt:
            logits = self.step(int(t))
        out, all_logits = [], []
        for _ in range(max_new_tokens):
            all_logits.append(logits)
            nxt = int(torch.argmax(logits))
            out.append(nxt)
            logits = self.step(nxt)
        return out, all_logits


# --------------------------------------------------------------------------------------
# native engine

# order = the engine's mode numbers
PREFILL_GEMMS = ("umma", "shadow", "fp8x2", "fp8")


class EngineError(RuntimeError):
    pass


class EngineSnapshot:
    """Device copy of the DeltaNet states and conv tails at one position. `update()` re-captures
    into the same buffers; `restore()` rewinds the engine (the KV cache is position indexed,
    so entries beyond the restored position are simply overwritten later)."""

    def __init__(self, engine: "QwenEngine", handle):
        self._e, self._s = engine, handle

    @property
    def position(self) -> int:
        return self._e._L.pk_qwen_snapshot_position(self._s)

    def update(self) -> None:
        self._e._ck(self._e._L.pk_qwen_snapshot_update(self._e._h, self._s))

    def restore(self) -> None:
        self._e._ck(self._e._L.pk_qwen_restore(self._e._h, self._s))

    def free(self) -> None:
        if self._s is not None and self._e._h:
            self._e._L.pk_qwen_free_snapshot(self._e._h, self._s)
        self._s = None


class QwenEngine:
    """Native engine for one tensor-parallel rank.

    `QwenEngine(cfg).load(path)` or `.init_random(seed)`, then `prefill(tokens)` followed
    by `decode(n)`. With `tp_world > 1` call `connect(...)` (see `parallel.tp`) once every
    rank has created its engine.
    """

    def __init__(self, cfg: QwenHybridConfig | str, *, tp_rank: int = 0, tp_world: int = 1, device: int = 0,
                 max_context: int = 4096, prefill_chunk: int = 512, use_cuda_graph: bool = True, decode_splits: int = 0,
                 mtp: bool = False, persistent_decode: int | None = None, kv_cache_dtype: str = "bf16",
                 prefill_gemm: str | None = None):
        """`persistent_decode`: 1 runs every single-row decode step as one persistent kernel, 0 as one launch per
        projection (the kernels that also serve verify rows, so speculative loops that compare tokens of the two must use
        0), None lets the engine choose. `kv_cache_dtype`: "bf16", or "fp8" (E4M3 codes with one scale per 64 channels: a little
        over half the bytes per cached position). `prefill_gemm`: how rows beyond eight are multiplied with the FP8 linears:
        "fp8x2" (default: tcgen05 FP8 math on the stored codes, activations as two E4M3 terms per value), "fp8" (one term:
        fastest, 4 significant bits per activation), "shadow" (bf16 copies of the weights in HBM) or "umma" (weights
        decoded to bf16 in shared memory)."""
        if prefill_gemm not in (None,) + PREFILL_GEMMS:
            raise ValueError(f"prefill_gemm must be one of {PREFILL_GEMMS}")
        if kv_cache_dtype not in ("bf16", "fp8"):
            raise ValueError("kv_cache_dtype must be 'bf16' or 'fp8'")
        self._L = _lib.engine()
        L = self._L
        L.pk_qwen_create_ex2.restype = ctypes.c_void_p
        L.pk_qwen_kv_cache_bytes.restype = ctypes.c_ulonglong
        L.pk_engine_last_error.restype = ctypes.c_char_p
        L.pk_qwen_comm_arena.restype = ctypes.c_void_p
        L.pk_qwen_weight_bytes.restype = ctypes.c_ulonglong
        L.pk_qwen_shadow_bytes.restype = ctypes.c_ulonglong
        L.pk_ipc_open.restype = ctypes.c_void_p
        L.pk_qwen_snapshot.restype = ctypes.c_void_p
        L.pk_qwen_snapshot_with_kv.restype = ctypes.c_void_p
        self.cfg = cfg
        text = cfg if isinstance(cfg, str) else cfg.to_json()
        self.tp_rank, self.tp_world, self.device = tp_rank, tp_world, device
        self.prefill_chunk = prefill_chunk
        self.mtp = bool(mtp)
        self.kv_cache_dtype = kv_cache_dtype
        self._h = L.pk_qwen_create_ex2(text.encode(), tp_rank, tp_world, device, max_context, prefill_chunk,
                                       int(use_cuda_graph), decode_splits, int(self.mtp), int(kv_cache_dtype == "fp8"))
        if not self._h:
            raise EngineError(L.pk_engine_last_error().decode())
        self._h = ctypes.c_void_p(self._h)
        if persistent_decode is not None:
            self._ck(L.pk_qwen_set_persistent_decode(self._h, int(persistent_decode)))
        if prefill_gemm is not None:
            self._ck(L.pk_qwen_set_prefill_gemm(self._h, PREFILL_GEMMS.index(prefill_gemm)))

    def _ck(self, status: int) -> None:
        if status != 0:
            raise EngineError(self._L.pk_engine_last_error().decode())

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._L.pk_qwen_destroy(self._h)
            self._h = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    def load(self, path: str | Path) -> "QwenEngine":
        self._ck(self._L.pk_qwen_load_safetensors(self._h, str(path).encode()))
        return self

    def init_random(self, seed: int = 0, sigma: float = 0.02) -> "QwenEngine":
        self._ck(self._L.pk_qwen_init_random(self._h, ctypes.c_uint64(seed), ctypes.c_float(sigma)))
        return self

    def reset(self) -> None:
        self._ck(self._L.pk_qwen_reset(self._h))

    def prefill(self, tokens: Sequence[int]) -> int:
        arr = (ctypes.c_int * len(tokens))(*[int(t) for t in tokens])
        first = ctypes.c_int(0)
        self._ck(self._L.pk_qwen_prefill(self._h, arr, len(tokens), ctypes.byref(first)))
        return first.value

    def prefill_reusing(self, tokens: Sequence[int]) -> tuple[int, dict]:
        """A new request with the engine's native prefix reuse: the KV cache is position indexed and stays between
        requests, the recurrent state continues live or rolls back to a stored copy (reference behaviour:
        cpp_engine/src/qwen_engine.cpp:662-826). Returns (first token, statistics)."""
        arr = (ctypes.c_int * len(tokens))(*[int(t) for t in tokens])
        first = ctypes.c_int(0)
        st = (ctypes.c_longlong * 9)()
        self._ck(self._L.pk_qwen_prefill_cached(self._h, arr, len(tokens), ctypes.byref(first), st))
        names = ("reused_tokens", "computed_tokens", "prompt_tokens", "matched_tokens", "source", "snapshots", "snapshot_bytes", "hits", "misses")
        d = dict(zip(names, (int(v) for v in st)))
        d["source"] = ("empty", "live", "snapshot")[d["source"]]
        return first.value, d

    def clear_prefix_cache(self) -> None:
        self._ck(self._L.pk_qwen_clear_prefix_cache(self._h))

    def configure_prefix_cache(self, enable: bool = True, snapshot_interval: int = 4096, max_snapshots: int = 82) -> None:
        self._ck(self._L.pk_qwen_configure_prefix_cache(self._h, int(enable), snapshot_interval, max_snapshots))

    def decode(self, steps: int, sync_each_step: bool = False) -> list[int]:
        out = (ctypes.c_int * steps)()
        self._ck(self._L.pk_qwen_decode(self._h, steps, out, int(sync_each_step)))
        return list(out)

    def forward_rows(self, tokens: Sequence[int]) -> list[int]:
        n = len(tokens)
        arr = (ctypes.c_int * n)(*[int(t) for t in tokens])
        out = (ctypes.c_int * n)()
        self._ck(self._L.pk_qwen_forward_rows(self._h, arr, n, out))
        return list(out)

    # -- multi-token predictor ------------------------------------------------------------
    def spec_decode(self, steps: int, max_draft: int = 4) -> tuple[list[int], dict[str, int]]:
        """`decode(steps)` with drafts from the model's own multi-token predictor (engine built with `mtp=True`),
        verified by the target in one multi-row pass per round: the same tokens, fewer target passes when drafts match.
        Returns (tokens, counters). Reference behaviour: cpp_engine/src/qwen_engine.cpp:1527-1553, 1646-1726, 2169-2270."""
        out = (ctypes.c_int * steps)()
        st = (ctypes.c_longlong * 7)()
        self._ck(self._L.pk_qwen_spec_decode(self._h, steps, max_draft, out, st))
        names = ("rounds", "proposed", "accepted", "rollbacks", "replay_tokens", "plain_steps", "predictor_rows")
        return list(out), dict(zip(names, (int(v) for v in st)))

    @property
    def mtp_next_token(self) -> int:
        """The predictor's pick for the token after `last_token` (-1 when it has to be rebuilt first)."""
        return self._L.pk_qwen_mtp_next_token(self._h)

    def mtp_logits(self) -> torch.Tensor:
        n = self._L.pk_qwen_vocab_local(self._h)
        buf = (ctypes.c_float * n)()
        self._ck(self._L.pk_qwen_copy_mtp_logits(self._h, buf))
        return torch.tensor(list(buf), dtype=torch.float32)

    def set_draft_replay(self, tokens: Sequence[int]) -> None:
        """Test hook: take drafts from a known continuation (the tokens after the first generated one); empty clears."""
        arr = (ctypes.c_int * max(len(tokens), 1))(*[int(t) for t in tokens])
        self._ck(self._L.pk_qwen_set_draft_replay(self._h, arr, len(tokens)))

    def generate_mtp(self, prompt: Sequence[int], max_new_tokens: int, max_draft: int = 4) -> tuple[list[int], dict[str, int]]:
        first = self.prefill(prompt)
        if max_new_tokens <= 1:
            return [first][:max_new_tokens], {}
        toks, stats = self.spec_decode(max_new_tokens - 1, max_draft)
        return [first] + toks, stats

    # -- recurrent-state snapshots (speculative decoding, prefix cache) -----------------
    def snapshot(self, with_kv: bool = False) -> "EngineSnapshot":
        """`with_kv` also keeps the KV rows before the current position, so that the snapshot stays valid after
        other requests have used the engine (prefix cache)."""
        h = (self._L.pk_qwen_snapshot_with_kv if with_kv else self._L.pk_qwen_snapshot)(self._h)
        if not h:
            raise EngineError(self._L.pk_engine_last_error().decode())
        return EngineSnapshot(self, ctypes.c_void_p(h))

    @property
    def position(self) -> int:
        return self._L.pk_qwen_position(self._h)

    @property
    def last_token(self) -> int:
        return self._L.pk_qwen_last_token(self._h)

    def generate_cached(self, prompt: Sequence[int], max_new_tokens: int, cache) -> tuple[list[int], int]:
        """`generate` through a `runtime.prefix_snapshot.PrefixSnapshotCache`: the longest cached prefix (whole blocks,
        at least one token left to run) is restored instead of recomputed, and the state at the last block boundary of
        this prompt is captured for later requests. Returns (tokens, number of prompt tokens that were reused)."""
        prompt = list(prompt)
        self.reset()
        hit = cache.restore(prompt)
        reused = 0
        if hit is not None:
            hit.state.restore()
            reused = hit.length
        boundary = (len(prompt) - 1) // cache.block * cache.block
        first = None
        if boundary > reused:
            self.prefill(prompt[reused:boundary])
            cache.capture(prompt[:boundary], self.snapshot(with_kv=True))
            reused_now = boundary
        else:
            reused_now = reused
        first = self.prefill(prompt[reused_now:])
        out = [first] if max_new_tokens <= 1 else [first] + self.decode(max_new_tokens - 1)
        return out[:max_new_tokens], reused

    def generate(self, prompt: Sequence[int], max_new_tokens: int) -> list[int]:
        first = self.prefill(prompt)
        if max_new_tokens <= 1:
            return [first][:max_new_tokens]
        return [first] + self.decode(max_new_tokens - 1)

    def logits(self, row: int = 0) -> torch.Tensor:
        n = self._L.pk_qwen_vocab_local(self._h)
        buf = (ctypes.c_float * n)()
        self._ck(self._L.pk_qwen_copy_logits(self._h, buf, row))
        return torch.tensor(list(buf), dtype=torch.float32)

    @property
    def weight_bytes(self) -> int:
        return int(self._L.pk_qwen_weight_bytes(self._h))

    @property
    def kv_cache_bytes(self) -> int:
        """Bytes of the K and V caches of every full-attention layer on this rank (scales included)."""
        return int(self._L.pk_qwen_kv_cache_bytes(self._h))

    def set_tap_layers(self, layers) -> None:
        """Capture the residual stream after each of `layers` for every row of every following forward (one rank only;
        decode steps then run one launch per projection). `taps()` reads them."""
        arr = (ctypes.c_int * len(layers))(*[int(v) for v in layers])
        self._ck(self._L.pk_qwen_set_tap_layers(self._h, arr, len(layers)))
        self._n_taps = len(layers)

    def taps(self, first_row: int = 0, rows: int | None = None) -> torch.Tensor:
        """bf16 [rows, taps * hidden] on the device: the taps of the last forward (prefill chunk, verify rows or decode step)."""
        total = int(self._L.pk_qwen_tap_rows(self._h))
        rows = total - first_row if rows is None else rows
        out = torch.empty(rows, self._n_taps * self.cfg.hidden_size, device=f"cuda:{self.device}", dtype=torch.bfloat16)
        self._ck(self._L.pk_qwen_copy_taps(self._h, ctypes.c_void_p(out.data_ptr()), first_row, rows))
        return out

    def verify_canaries(self) -> None:
        """With POCKET_CANARY=1 in the environment when the engine was created, every device buffer has guard bytes on both
        sides; raises EngineError naming the first buffer whose guards were overwritten."""
        if not self._L.pk_qwen_canaries_enabled(self._h):
            raise EngineError("canaries are off: set POCKET_CANARY=1 before creating the engine")
        if self._L.pk_qwen_verify_canaries(self._h) != -1:
            raise EngineError(self._L.pk_engine_last_error().decode())

    def enable_nccl_fallback(self, id_path: str, timeout_ms: int = 600000) -> None:
        """Join the group's NCCL communicator (every rank calls this; file rendezvous under `id_path`). From then on a
        step that fails on a bounded peer wait still raises, and all later steps run their collectives through NCCL."""
        self._ck(self._L.pk_qwen_enable_nccl_fallback(self._h, str(id_path).encode(), int(timeout_ms)))

    def switch_to_nccl(self) -> None:
        """Leave the peer-store path now (a rank that learnt of another rank's failure on the host)."""
        self._ck(self._L.pk_qwen_switch_to_nccl(self._h))

    @property
    def nccl_mode(self) -> bool:
        return bool(self._L.pk_qwen_nccl_mode(self._h))

    def set_comm_timeout_us(self, us: int) -> None:
        """Budget of every device-side wait on a peer."""
        self._ck(self._L.pk_qwen_set_comm_timeout_us(self._h, int(us)))

    @property
    def prefill_gemm(self) -> str:
        """The GEMM that multiplies more than eight rows with the FP8 linears (known once the weights are in place)."""
        return PREFILL_GEMMS[int(self._L.pk_qwen_prefill_gemm_mode(self._h))]

    @property
    def prefill_shadow_bytes(self) -> int:
        """Bytes of the bf16 weight copies used by the tensor-core prefill path (0 when off)."""
        return int(self._L.pk_qwen_shadow_bytes(self._h))

    @property
    def persistent_decode(self) -> bool:
        """True when single-row decode steps run as one persistent kernel per token (known after the first `decode`).
        `POCKET_DECODE_PERSISTENT=0` in the environment keeps one launch per projection."""
        return bool(self._L.pk_qwen_persistent_decode_active(self._h))

    PHASE_NAMES = {0: "start", 1: "stage_norm", 8: "stage_plain", 9: "stage_headnorm", 10: "in_proj", 11: "in_proj_ab", 12: "out_proj",
                   13: "gate_up", 14: "down", 20: "lm_head", 3: "grid_barrier", 4: "site_barrier", 5: "deltanet", 6: "attn_split",
                   7: "attn_merge"}

    def decode_trace(self) -> dict[str, float]:
        """Microseconds block 0 spent per phase kind in the last persistent decode step (engine created with
        `POCKET_DECODE_TRACE=1` in the environment); empty otherwise."""
        cap = 4096
        buf = (ctypes.c_ulonglong * (2 * cap))()
        n = self._L.pk_qwen_decode_trace(self._h, buf, cap)
        out: dict[str, float] = {}
        for i in range(1, n):
            name = self.PHASE_NAMES.get(int(buf[2 * i]), str(int(buf[2 * i])))
            out[name] = out.get(name, 0.0) + (buf[2 * i + 1] - buf[2 * i - 1]) / 1e3
        if n > 1:
            out["total"] = (buf[2 * n - 1] - buf[1]) / 1e3
        return out

    def comm_status(self) -> int:
        return int(self._L.pk_qwen_comm_status(self._h)) & 0xFFFFFFFF

    def timings(self) -> dict[str, float]:
        buf = (ctypes.c_double * 5)()
        self._L.pk_qwen_timings(self._h, buf)
        return {"prefill_ms": buf[0], "decode_ms": buf[1], "prefill_tokens": buf[2], "decode_tokens": buf[3],
                "kernel_launches": buf[4]}

    # ---- peer memory ----
    def export_arena(self) -> bytes:
        n = ctypes.c_ulonglong(0)
        ptr = self._L.pk_qwen_comm_arena(self._h, ctypes.byref(n))
        handle = (ctypes.c_ubyte * 64)()
        self._ck(self._L.pk_ipc_export(ctypes.c_void_p(ptr), handle))
        return bytes(handle)

    def connect(self, handles: Sequence[bytes]) -> None:
        """Register the comm arenas of all ranks (`handles[r]` from rank r's `export_arena`)."""
        ptrs = (ctypes.c_void_p * self.tp_world)()
        for r, hb in enumerate(handles):
            if r == self.tp_rank:
                ptrs[r] = None
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(hb)
            p = self._L.pk_ipc_open(buf)
            if not p:
                raise EngineError(self._L.pk_engine_last_error().decode())
            ptrs[r] = p
        self._ck(self._L.pk_qwen_set_peer_arenas(self._h, ptrs))
