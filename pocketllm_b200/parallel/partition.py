"""Partition policies: which rank holds which slice of which checkpoint tensor.

One rule table serves every checkpoint format, so a weight lands on the same rank whether it
comes from Safetensors or GGUF. Policies (the reference's `legacy`, `baseline_4gpu`,
`layer_pp_4gpu`, src/models/deepseek_v4/partition.py:17-58,154-270, generalised to 1..8
ranks of one NVSwitch node):

* `replicated` - every rank holds everything except routed experts outside its range.
* `tp`         - column-parallel tensors split on dim 0, row-parallel on dim 1, attention
                 sinks on dim 0, routed experts by contiguous range, the rest replicated.
* `layer_pp`   - contiguous layer ranges per stage; embedding on the first stage, final norm,
                 head and MTP blocks on the last.

Rules are decided from tensor names (a regular-expression table) rather than from module
classes, so loaders can plan reads before any module exists.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass

import numpy as np

POLICIES = ("replicated", "tp", "layer_pp")
ALIASES = {"legacy": "replicated", "baseline_4gpu": "tp", "layer_pp_4gpu": "layer_pp", None: "replicated"}

# Run-time modes that break "each rank owns a balanced contiguous slice"; refusing to start
# beats a silently degenerate layout.
FORBIDDEN_WITH_SHARDED = ("POCKET_CPU_MOE_INPROC_SERVER", "POCKET_CPU_MOE_RANK0_SERVER", "POCKET_REPLICATED_INDEXER")

_COLUMN = re.compile(r"(^embed\.|^head\.|\.(wq_b|wkv_b|wq|wk|wv|w1|w3|gate_proj|up_proj|q_proj|k_proj|v_proj|weights_proj)\.(weight|scale)$)")
_ROW = re.compile(r"\.(wo|wo_b|w2|down_proj|o_proj)\.(weight|scale)$")
_EXPERT = re.compile(r"(?:^|\.)experts\.(\d+)\.")


def normalize_policy(policy: str | None) -> str:
    p = ALIASES.get(policy, policy)
    if p not in POLICIES:
        raise ValueError(f"unsupported partition policy {policy!r}; expected one of {POLICIES}")
    return p


def _truthy(name: str) -> bool:
    return os.environ.get(name, "0").lower() in ("1", "true", "yes")


def check_environment(policy: str, world: int) -> None:
    policy = normalize_policy(policy)
    if policy == "replicated":
        return
    bad = [n for n in FORBIDDEN_WITH_SHARDED if _truthy(n)]
    if not 1 <= world <= 8:
        bad.append(f"world_size={world}")
    if policy == "layer_pp" and _truthy("POCKET_DECODE_MTP_SPEC"):
        bad.append("POCKET_DECODE_MTP_SPEC")
    if bad:
        raise RuntimeError(f"partition policy {policy} is incompatible with: {', '.join(bad)}")


def expert_index(name: str) -> int | None:
    if "shared_experts" in name:
        return None
    m = _EXPERT.search(name)
    return int(m.group(1)) if m else None


def expert_range(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    return rank * n_experts // world, (rank + 1) * n_experts // world


def rule_kind(name: str) -> str:
    if expert_index(name) is not None:
        return "expert_owned"
    if "shared_experts" in name:
        return "replicated_shared_expert"
    if name.endswith("attn_sink"):
        return "attn_sink"
    if _ROW.search(name):
        return "row_parallel"
    if _COLUMN.search(name):
        return "column_parallel"
    return "replicated"


@dataclass(frozen=True)
class Shard:
    """`dim is None`: the whole tensor; `owned False`: this rank reads nothing."""
    owned: bool
    dim: int | None = None
    start: int = 0
    size: int = 0


def shard_for_rank(name: str, shape: tuple[int, ...], policy: str, world: int, rank: int, *, n_experts: int = 0, n_layers: int = 0) -> Shard:
    policy = normalize_policy(policy)
    if policy == "layer_pp":
        owner = parameter_owner(name, n_layers, world)
        return Shard(owner is None or owner == rank)
    kind = rule_kind(name)
    if kind == "expert_owned":
        lo, hi = expert_range(n_experts, world, rank) if n_experts else (0, 1 << 30)
        return Shard(lo <= expert_index(name) < hi)
    if policy == "replicated" or world == 1:
        return Shard(True)
    dim = {"column_parallel": 0, "attn_sink": 0, "row_parallel": 1}.get(kind)
    if dim is None or len(shape) <= dim or (kind == "row_parallel" and len(shape) != 2):
        return Shard(True)
    if shape[dim] % world:
        raise ValueError(f"{name}: shape {shape} is not divisible by {world} on dim {dim}")
    n = shape[dim] // world
    return Shard(True, dim, rank * n, n)


def shard_tensor(name: str, tensor, policy: str, world: int, rank: int, **kw):
    """The rank-local slice (a contiguous copy), the tensor itself, or None when not owned."""
    s = shard_for_rank(name, tuple(tensor.shape), policy, world, rank, **kw)
    if not s.owned:
        return None
    if s.dim is None:
        return tensor
    if isinstance(tensor, np.ndarray):
        idx = [slice(None)] * tensor.ndim
        idx[s.dim] = slice(s.start, s.start + s.size)
        return np.ascontiguousarray(tensor[tuple(idx)])
    return tensor.narrow(s.dim, s.start, s.size).contiguous()


def shard_quant_blocks(name: str, blocks, policy: str, world: int, rank: int, **kw):
    """Quantised tensors as `[rows, blocks_per_row, block_bytes]`: column-parallel splits rows,
    row-parallel splits whole blocks along K (a block never straddles two ranks)."""
    s = shard_for_rank(name, tuple(blocks.shape[:2]), policy, world, rank, **kw)
    if not s.owned:
        return None
    if s.dim is None:
        return blocks
    return _narrow(blocks, s)


def _narrow(t, s: Shard):
    if isinstance(t, np.ndarray):
        idx = [slice(None)] * t.ndim
        idx[s.dim] = slice(s.start, s.start + s.size)
        return np.ascontiguousarray(t[tuple(idx)])
    return t.narrow(s.dim, s.start, s.size).contiguous()


def layer_range(n_layers: int, stages: int, stage: int) -> tuple[int, int]:
    return stage * n_layers // stages, (stage + 1) * n_layers // stages


def layer_owner(layer: int, n_layers: int, stages: int) -> int:
    if not 0 <= layer < n_layers:
        raise ValueError(f"layer {layer} out of range for {n_layers} layers")
    for s in range(stages):
        lo, hi = layer_range(n_layers, stages, s)
        if lo <= layer < hi:
            return s
    raise AssertionError


def parameter_owner(name: str, n_layers: int, stages: int) -> int | None:
    """Owning stage, or None for tensors every stage keeps."""
    if name.startswith("embed."):
        return 0
    if name.startswith(("norm.", "head.", "hc_head_", "mtp.")):
        return stages - 1
    m = re.match(r"layers\.(\d+)\.", name)
    if m:
        return layer_owner(int(m.group(1)), n_layers, stages)
    return None


def needed_keys(keys, policy: str, world: int, rank: int, *, n_experts: int = 0, n_layers: int = 0) -> list[str]:
    """Checkpoint keys this rank must read. A `.scale` travels with its `.weight`."""
    ks = set(keys)
    out = []
    for k in keys:
        if k.endswith(".scale") and k[:-6] + ".weight" in ks:
            continue
        if shard_for_rank(k, (), policy, world, rank, n_experts=n_experts, n_layers=n_layers).owned:
            out.append(k)
    return out


def layout_line(policy: str, world: int, rank: int, *, vocab: int = 0, n_heads: int = 0, n_experts: int = 0, n_layers: int = 0) -> str:
    """One grep-able line per rank describing the realised layout."""
    policy = normalize_policy(policy)
    if policy == "layer_pp":
        lo, hi = layer_range(n_layers, world, rank)
        return (f"partition_layout policy={policy} world_size={world} rank={rank} pp_rank={rank} pp_size={world} tp_size=1 "
                f"layers=[{lo},{hi}) owns_embed={rank == 0} owns_head={rank == world - 1} expert_range=0:{n_experts}")
    tp = world if policy == "tp" else 1
    r = rank if policy == "tp" else 0
    elo, ehi = expert_range(n_experts, world, rank) if n_experts else (0, 0)
    return (f"partition_layout policy={policy} world_size={world} rank={rank} vocab=[{r * vocab // tp},{(r + 1) * vocab // tp}) "
            f"local_heads={n_heads // tp} expert_range={elo}:{ehi}")
