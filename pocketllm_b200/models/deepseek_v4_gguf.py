"""DeepSeek-V4 from GGUF (`general.architecture = deepseek4`): tensor naming, writer for synthetic files and loader.

GGUF tensor names (reference: src/loader/mappings/deepseek_v4.py:58-140): `token_embd`, `output`, `output_norm`,
`output_hc_{fn,base,scale}`; per layer `blk.L.attn_{sinks,q_a,q_a_norm,q_b,kv,kv_a_norm,output_a,output_b,norm}`,
`ffn_gate_inp`, `ffn_gate_tid2eid` (hash layers) or `exp_probs_b.bias`, `ffn_{gate,down,up}_exps` [E, N, K],
`ffn_{gate,down,up}_shexp`, `ffn_norm`, `hc_{attn,ffn}_{fn,base,scale}`, `attn_compressor_{ape,kv,gate,norm}`,
`indexer.attn_q_b`, `indexer.proj`, `indexer_compressor_{ape,kv,gate,norm}`.

Dense matrices (Q8_0 in the published files) are dequantised at load; routed experts stay in their GGUF block format in
HBM and run through the in-register decoders, so IQ2_XXS / Q2_K / IQ1_M / Q4_K expert files work unchanged.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from ..formats import gguf
from ..formats import gguf_quants as gq
from . import deepseek_v4 as d4

ARCH = "deepseek4"

_LAYER = {  # gguf suffix -> (target suffix, is a quantisable matrix)
    "attn_sinks.weight": ("attn.attn_sink", False), "attn_q_a.weight": ("attn.wq_a.weight", True),
    "attn_q_a_norm.weight": ("attn.q_norm.weight", False), "attn_q_b.weight": ("attn.wq_b.weight", True),
    "attn_kv.weight": ("attn.wkv.weight", True), "attn_kv_a_norm.weight": ("attn.kv_norm.weight", False),
    "attn_output_a.weight": ("attn.wo_a.weight", True), "attn_output_b.weight": ("attn.wo_b.weight", True),
    "attn_norm.weight": ("attn_norm.weight", False), "ffn_gate_inp.weight": ("ffn.gate.weight", False),
    "ffn_gate_tid2eid.weight": ("ffn.gate.tid2eid", False), "exp_probs_b.bias": ("ffn.gate.bias", False),
    "ffn_gate_shexp.weight": ("ffn.shared_experts.w1.weight", True), "ffn_down_shexp.weight": ("ffn.shared_experts.w2.weight", True),
    "ffn_up_shexp.weight": ("ffn.shared_experts.w3.weight", True), "ffn_norm.weight": ("ffn_norm.weight", False),
    "hc_attn_fn.weight": ("hc_attn_fn", False), "hc_attn_base.weight": ("hc_attn_base", False), "hc_attn_scale.weight": ("hc_attn_scale", False),
    "hc_ffn_fn.weight": ("hc_ffn_fn", False), "hc_ffn_base.weight": ("hc_ffn_base", False), "hc_ffn_scale.weight": ("hc_ffn_scale", False),
    "attn_compressor_ape.weight": ("attn.compressor.ape", False), "attn_compressor_kv.weight": ("attn.compressor.wkv.weight", False),
    "attn_compressor_gate.weight": ("attn.compressor.wgate.weight", False), "attn_compressor_norm.weight": ("attn.compressor.norm.weight", False),
    "indexer.attn_q_b.weight": ("attn.indexer.wq_b.weight", True), "indexer.proj.weight": ("attn.indexer.weights_proj.weight", False),
    "indexer_compressor_ape.weight": ("attn.indexer.compressor.ape", False), "indexer_compressor_kv.weight": ("attn.indexer.compressor.wkv.weight", False),
    "indexer_compressor_gate.weight": ("attn.indexer.compressor.wgate.weight", False),
    "indexer_compressor_norm.weight": ("attn.indexer.compressor.norm.weight", False),
}
_TOP = {"token_embd.weight": ("embed.weight", True), "output.weight": ("head.weight", True), "output_norm.weight": ("norm.weight", False),
        "output_hc_fn.weight": ("hc_head_fn", False), "output_hc_base.weight": ("hc_head_base", False), "output_hc_scale.weight": ("hc_head_scale", False)}
_EXPERT_PART = {"gate": "w1", "up": "w3", "down": "w2"}


def metadata(cfg: d4.DSV4Config) -> dict:
    return {"general.architecture": ARCH, f"{ARCH}.block_count": cfg.n_layers, f"{ARCH}.hash_layer_count": cfg.n_hash_layers,
            f"{ARCH}.expert_count": cfg.n_routed_experts, f"{ARCH}.expert_used_count": cfg.n_activated_experts,
            f"{ARCH}.embedding_length": cfg.dim, f"{ARCH}.context_length": cfg.max_seq_len, f"{ARCH}.vocab_size": cfg.vocab_size,
            f"{ARCH}.pocket_config": cfg.to_json()}


def config_from_metadata(md: dict) -> d4.DSV4Config:
    if md.get("general.architecture") != ARCH:
        raise ValueError(f"not a {ARCH} GGUF: {md.get('general.architecture')!r}")
    if f"{ARCH}.pocket_config" in md:
        return d4.DSV4Config.from_json(md[f"{ARCH}.pocket_config"])
    # Published files carry only the counts; everything else is the V4-Flash shape.
    return d4.DSV4Config(n_layers=int(md.get(f"{ARCH}.block_count", 43)), n_hash_layers=int(md.get(f"{ARCH}.hash_layer_count", 3)),
                         n_routed_experts=int(md.get(f"{ARCH}.expert_count", 256)), n_activated_experts=int(md.get(f"{ARCH}.expert_used_count", 6)),
                         dim=int(md.get(f"{ARCH}.embedding_length", 4096)), vocab_size=int(md.get(f"{ARCH}.vocab_size", 129280)), n_mtp_layers=0)


def tensor_plan(cfg: d4.DSV4Config, dense_type: str = "q8_0", expert_type: str = "q4_k") -> list[tuple[str, tuple[int, ...], str]]:
    """(gguf name, torch-order shape, type) of every tensor of a deepseek4 GGUF (MTP blocks are not stored in GGUF)."""
    plan: list[tuple[str, tuple[int, ...], str]] = []
    d, hd, H, ql = cfg.dim, cfg.head_dim, cfg.n_heads, cfg.q_lora_rank
    q = lambda k: dense_type if k % 32 == 0 else "f32"
    plan += [("token_embd.weight", (cfg.vocab_size, d), q(d)), ("output.weight", (cfg.vocab_size, d), q(d)), ("output_norm.weight", (d,), "f32"),
             ("output_hc_fn.weight", (cfg.hc_mult, cfg.hc_mult * d), "f32"), ("output_hc_base.weight", (cfg.hc_mult,), "f32"),
             ("output_hc_scale.weight", (1,), "f32")]
    for l in range(cfg.n_layers):
        b, ratio = f"blk.{l}.", cfg.ratio(l)
        plan += [(b + "attn_sinks.weight", (H,), "f32"), (b + "attn_q_a.weight", (ql, d), q(d)), (b + "attn_q_a_norm.weight", (ql,), "f32"),
                 (b + "attn_q_b.weight", (H * hd, ql), q(ql)), (b + "attn_kv.weight", (hd, d), q(d)), (b + "attn_kv_a_norm.weight", (hd,), "f32"),
                 (b + "attn_output_a.weight", (cfg.o_groups * cfg.o_lora_rank, H * hd // cfg.o_groups), q(H * hd // cfg.o_groups)),
                 (b + "attn_output_b.weight", (d, cfg.o_groups * cfg.o_lora_rank), q(cfg.o_groups * cfg.o_lora_rank)), (b + "attn_norm.weight", (d,), "f32"),
                 (b + "ffn_gate_inp.weight", (cfg.n_routed_experts, d), "f32"), (b + "ffn_norm.weight", (d,), "f32")]
        plan.append((b + "ffn_gate_tid2eid.weight", (cfg.vocab_size, cfg.n_activated_experts), "i32") if l < cfg.n_hash_layers
                    else (b + "exp_probs_b.bias", (cfg.n_routed_experts,), "f32"))
        E, I = cfg.n_routed_experts, cfg.moe_inter_dim
        plan += [(b + "ffn_gate_exps.weight", (E, I, d), expert_type), (b + "ffn_up_exps.weight", (E, I, d), expert_type),
                 (b + "ffn_down_exps.weight", (E, d, I), expert_type)]
        si = cfg.n_shared_experts * I
        plan += [(b + "ffn_gate_shexp.weight", (si, d), q(d)), (b + "ffn_up_shexp.weight", (si, d), q(d)), (b + "ffn_down_shexp.weight", (d, si), q(si))]
        for kind in ("attn", "ffn"):
            plan += [(b + f"hc_{kind}_fn.weight", (cfg.mix_hc, cfg.hc_mult * d), "f32"), (b + f"hc_{kind}_base.weight", (cfg.mix_hc,), "f32"),
                     (b + f"hc_{kind}_scale.weight", (3,), "f32")]
        if ratio:
            coff = 2 if ratio == 4 else 1
            plan += [(b + "attn_compressor_ape.weight", (ratio, coff * hd), "f32"), (b + "attn_compressor_kv.weight", (coff * hd, d), "f32"),
                     (b + "attn_compressor_gate.weight", (coff * hd, d), "f32"), (b + "attn_compressor_norm.weight", (hd,), "f32")]
        if ratio == 4:
            ih, idim = cfg.index_n_heads, cfg.index_head_dim
            plan += [(b + "indexer.attn_q_b.weight", (ih * idim, ql), q(ql)), (b + "indexer.proj.weight", (ih, d), "f32"),
                     (b + "indexer_compressor_ape.weight", (4, 2 * idim), "f32"), (b + "indexer_compressor_kv.weight", (2 * idim, d), "f32"),
                     (b + "indexer_compressor_gate.weight", (2 * idim, d), "f32"), (b + "indexer_compressor_norm.weight", (idim,), "f32")]
    return plan


def _target(name: str) -> str:
    if name in _TOP:
        return _TOP[name][0]
    _, l, suffix = name.split(".", 2)
    return f"layers.{l}.{_LAYER[suffix][0]}"


def write_gguf(path: str | Path, cfg: d4.DSV4Config, W: dict[str, torch.Tensor], dense_type: str = "q8_0", expert_type: str = "q4_k") -> None:
    """Write `W` (the oracle's fp32 / FP4 weight dict) as a deepseek4 GGUF, quantising dense matrices and routed experts."""
    w = gguf.GGUFWriter()
    for k, v in metadata(cfg).items():
        w.add_meta(k, v)
    for name, shape, typ in tensor_plan(cfg, dense_type, expert_type):
        m = name.split(".")
        if len(m) > 2 and m[2].startswith("ffn_") and m[2].endswith("_exps"):
            part = _EXPERT_PART[m[2][4:-5]]
            mats = np.stack([d4.expert_weight(W, f"layers.{m[1]}.ffn.experts.{e}.{part}").numpy() for e in range(shape[0])])
            w.add_tensor(name, gq.quantize(mats.reshape(-1, shape[-1]), typ).reshape(*shape[:-1], -1) if typ not in ("f32", "f16") else mats.astype(np.float32), typ, shape)
            continue
        t = W[_target(name)]
        if typ == "i32":
            w.add_tensor(name, t.to(torch.int32).numpy(), "i32", shape)
        elif typ == "f32":
            w.add_tensor(name, t.float().numpy().reshape(shape), "f32", shape)
        else:
            w.add_tensor(name, gq.quantize(t.float().numpy(), typ), typ, shape)
    w.write(path)


def load_gguf(path: str | Path) -> tuple[d4.DSV4Config, dict[str, torch.Tensor], dict[str, tuple[torch.Tensor, str]]]:
    """(config, dense weights as fp32 under the oracle's names, raw routed experts).
    The third value maps `layers.L.ffn.{w13,w2}` to (uint8 [E, bytes per expert], ggml type name): per expert the gate rows,
    then the up rows (w13), or the down rows (w2), exactly as stored."""
    b = gguf.GGUFBundle(path)
    cfg = config_from_metadata(b.metadata)
    W: dict[str, torch.Tensor] = {}
    raw: dict[str, tuple[torch.Tensor, str]] = {}
    for name, t in b.tensors.items():
        parts = name.split(".")
        if len(parts) > 2 and parts[2] in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
            continue
        if t.type_name == "i32":
            W[_target(name)] = torch.from_numpy(np.frombuffer(b.raw(name), dtype=np.int32).reshape(t.shape).copy())
        else:
            W[_target(name)] = torch.from_numpy(gq.dequantize(b.blocks(name), t.type_name).reshape(t.shape).copy())
    for l in range(cfg.n_layers):
        g, u, dn = (b.tensors[f"blk.{l}.ffn_{k}_exps.weight"] for k in ("gate", "up", "down"))
        if g.type_name != u.type_name:
            raise ValueError(f"layer {l}: gate and up experts use different block formats")
        E = g.shape[0]
        gb = np.ascontiguousarray(b.blocks(f"blk.{l}.ffn_gate_exps.weight")).reshape(E, -1)
        ub = np.ascontiguousarray(b.blocks(f"blk.{l}.ffn_up_exps.weight")).reshape(E, -1)
        raw[f"layers.{l}.ffn.w13"] = (torch.from_numpy(np.concatenate([gb, ub], 1)), g.type_name)
        raw[f"layers.{l}.ffn.w2"] = (torch.from_numpy(np.ascontiguousarray(b.blocks(f"blk.{l}.ffn_down_exps.weight")).reshape(E, -1).copy()), dn.type_name)
    return cfg, W, raw


def dense_experts(path: str | Path, W: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """`W` plus every routed expert dequantised to fp32 under `layers.L.ffn.experts.E.wN.weight` (for the oracle)."""
    b = gguf.GGUFBundle(path)
    cfg = config_from_metadata(b.metadata)
    out = dict(W)
    for l in range(cfg.n_layers):
        for k, part in _EXPERT_PART.items():
            name = f"blk.{l}.ffn_{k}_exps.weight"
            mats = gq.dequantize(b.blocks(name), b.tensors[name].type_name).reshape(b.tensors[name].shape)
            for e in range(mats.shape[0]):
                out[f"layers.{l}.ffn.experts.{e}.{part}.weight"] = torch.from_numpy(mats[e].copy())
    return out
