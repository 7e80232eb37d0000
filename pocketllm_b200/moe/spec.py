"""Model specs for GGUF MoE checkpoints: parameters parsed from metadata, expected tensors,
validation, quantisation capability and placement reports.

Roles of the reference's `MoEModelSpec` protocol, `MoEArchitectureParams`, `SpecValidation`,
`CapabilityReport` and placement decisions (src/components/moe/{spec,capability,placement,
registry}.py), with the hardware profile of one 8xB200 node instead of 4x22 GiB cards.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..formats import gguf

# block types every kernel path can decode in place
SUPPORTED_QUANTS = ("f32", "f16", "bf16", "i32", "q8_0", "q2_k", "q4_k", "q5_k", "q6_k", "iq1_m", "iq2_xxs", "iq2_xs", "iq3_xxs", "iq4_xs")


@dataclass
class MoEArchitectureParams:
    architecture: str
    n_layers: int
    hidden_size: int
    vocab_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    n_routed_experts: int
    top_k: int
    expert_intermediate_size: int
    n_shared_experts: int = 0
    leading_dense_layers: int = 0
    context_length: int = 0
    rope_dim: int = 0
    rope_base: float = 0.0
    norm_eps: float = 1e-6


@dataclass
class SpecValidation:
    ok: bool
    missing: list[str] = field(default_factory=list)
    wrong_shape: list[str] = field(default_factory=list)
    unexpected_types: list[str] = field(default_factory=list)

    def summary(self) -> str:
        if self.ok:
            return "spec validation: ok"
        return (f"spec validation: FAILED missing={len(self.missing)} wrong_shape={len(self.wrong_shape)} "
                f"unexpected_types={len(self.unexpected_types)}")


@dataclass
class CapabilityReport:
    per_type_bytes: dict[str, int]
    unsupported: list[str]
    total_bytes: int

    @property
    def supported(self) -> bool:
        return not self.unsupported


@dataclass
class HardwareProfile:
    """One node: `n_gpus` devices of `hbm_gib` each, `reserve_fraction` kept free for
    activations, KV and workspaces."""
    n_gpus: int = 8
    hbm_gib: float = 180.0
    reserve_fraction: float = 0.15
    host_pinned_gib: float = 1024.0


@dataclass
class PlacementReport:
    mode: str                   # "resident" | "host_staged" | "does_not_fit"
    per_gpu_gib: float
    budget_gib: float
    expert_gib_total: float
    dense_gib_total: float
    resident_experts_per_gpu: int
    note: str = ""


def _plan_for(arch: str, md: dict):
    if arch == "minimax-m2":
        from ..models import minimax_m2 as m
        cfg = m.MiniMaxM2Config.from_gguf(md)
        return cfg, m.tensor_plan(cfg)
    if arch == "glm-dsa":
        from ..models import glm_dsa as m
        cfg = m.GLMDSAConfig.from_gguf(md)
        return cfg, m.tensor_plan(cfg)
    if arch == "deepseek4":
        from ..models import deepseek_v4_gguf as m
        cfg = m.config_from_metadata(md)
        return cfg, m.tensor_plan(cfg)
    raise KeyError(f"no spec for architecture {arch!r}")


def parse_params(bundle: gguf.GGUFBundle) -> MoEArchitectureParams:
    arch = bundle.architecture()
    cfg, _ = _plan_for(arch, bundle.metadata)
    if arch == "minimax-m2":
        return MoEArchitectureParams(arch, cfg.n_layers, cfg.dim, cfg.vocab_size, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim,
                                     cfg.n_experts, cfg.n_experts_used, cfg.expert_inter, 0, 0,
                                     int(bundle.metadata.get(arch + ".context_length", 0)), cfg.rope_dim, cfg.rope_theta, cfg.norm_eps)
    if arch == "deepseek4":
        return MoEArchitectureParams(arch, cfg.n_layers, cfg.dim, cfg.vocab_size, cfg.n_heads, 1, cfg.head_dim, cfg.n_routed_experts,
                                     cfg.n_activated_experts, cfg.moe_inter_dim, cfg.n_shared_experts, 0, cfg.max_seq_len, cfg.rope_head_dim,
                                     cfg.rope_theta, cfg.norm_eps)
    return MoEArchitectureParams(arch, cfg.n_layers, cfg.dim, cfg.vocab_size, cfg.n_heads, 1, cfg.key_mla_dim, cfg.n_experts, cfg.top_k,
                                 cfg.expert_inter, cfg.n_shared, cfg.leading_dense_layers,
                                 int(bundle.metadata.get(arch + ".context_length", 0)), cfg.rope_dim, cfg.rope_theta, cfg.norm_eps)


def validate(bundle: gguf.GGUFBundle) -> SpecValidation:
    """Every planned tensor exists with the planned shape; quantised tensors may use any supported type."""
    _, plan = _plan_for(bundle.architecture(), bundle.metadata)
    v = SpecValidation(True)
    have = bundle.tensors
    for name, shape, typ in plan:
        if name not in have:
            v.missing.append(name)
            continue
        t = have[name]
        if tuple(t.shape) != tuple(shape):
            v.wrong_shape.append(f"{name}: {tuple(t.shape)} != {tuple(shape)}")
        if t.type_name not in SUPPORTED_QUANTS or (typ in ("f32", "i32") and t.type_name != typ):
            v.unexpected_types.append(f"{name}: {t.type_name}")
    v.ok = not (v.missing or v.wrong_shape or v.unexpected_types)
    return v


def capability(bundle: gguf.GGUFBundle) -> CapabilityReport:
    per: dict[str, int] = {}
    for t in bundle.tensors.values():
        per[t.type_name] = per.get(t.type_name, 0) + t.nbytes
    return CapabilityReport(per, sorted(k for k in per if k not in SUPPORTED_QUANTS), sum(per.values()))


def placement(bundle: gguf.GGUFBundle, hw: HardwareProfile | None = None, world: int | None = None) -> PlacementReport:
    """Experts are split over the ranks (contiguous ranges), dense weights are replicated."""
    hw = hw or HardwareProfile()
    world = world or hw.n_gpus
    gib = float(1 << 30)
    expert = sum(t.nbytes for n, t in bundle.tensors.items() if "_exps." in n) / gib
    dense = sum(t.nbytes for n, t in bundle.tensors.items() if "_exps." not in n) / gib
    budget = hw.hbm_gib * (1.0 - hw.reserve_fraction)
    per_gpu = dense + expert / world
    n_exp = parse_params(bundle).n_routed_experts
    if per_gpu <= budget:
        return PlacementReport("resident", per_gpu, budget, expert, dense, n_exp // world)
    room = max(budget - dense, 0.0)
    if dense < budget and expert <= hw.host_pinned_gib:
        per_expert = expert / max(n_exp, 1)
        return PlacementReport("host_staged", dense + room, budget, expert, dense, int(room / max(per_expert * 1.0, 1e-9)) // 1,
                               "experts beyond the resident set are staged from pinned host memory on a side stream")
    return PlacementReport("does_not_fit", per_gpu, budget, expert, dense, 0, "dense weights alone exceed the per-GPU budget")
