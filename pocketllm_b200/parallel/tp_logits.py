"""Vocabulary-sharded logits across tensor-parallel ranks: row ranges, distributed greedy argmax and
gather of the full row (reference: src/components/gguf/tp_logits.py:29-55)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def vocab_row_range(vocab: int, world: int, rank: int) -> tuple[int, int]:
    """Rows of the output head owned by `rank`: equal shares of ceil(vocab / world), the last one short."""
    per = (vocab + world - 1) // world
    return min(rank * per, vocab), min((rank + 1) * per, vocab)


def distributed_argmax(local_logits: torch.Tensor, vocab: int, group=None) -> torch.Tensor:
    """Greedy token per row from logits sharded on the last dim. Ties go to the lowest token id on every rank alike."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    lo, _ = vocab_row_range(vocab, world, rank)
    val, idx = local_logits.float().max(-1)
    pair = torch.stack([val, (idx + lo).float()], -1).contiguous()
    allp = [torch.empty_like(pair) for _ in range(world)]
    dist.all_gather(allp, pair, group=group)
    allp = torch.stack(allp, 0)                                    # [world, rows, 2]
    best = allp[..., 0].max(0)[0]
    ids = torch.where(allp[..., 0] == best, allp[..., 1], torch.full_like(allp[..., 1], float(vocab)))
    return ids.min(0)[0].long()


def gather_logits(local_logits: torch.Tensor, vocab: int, group=None) -> torch.Tensor:
    """Full [rows, vocab] logits on every rank (shards are padded to equal size for the collective)."""
    world = dist.get_world_size(group)
    per = (vocab + world - 1) // world
    pad = local_logits.new_full((*local_logits.shape[:-1], per), float("-inf"))
    pad[..., : local_logits.shape[-1]] = local_logits
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad.contiguous(), group=group)
    return torch.cat(parts, -1)[..., :vocab]
