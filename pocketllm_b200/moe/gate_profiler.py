"""Cross-layer gate statistics: how many of a layer's routed experts were already predicted from the
previous layer's hidden state, expert load histograms and overlap between consecutive layers
(reference: the cross-layer gate profiler in src/models/deepseek_v4/runtime.py:314-419)."""
from __future__ import annotations

from collections import defaultdict

import torch


class GateProfiler:
    def __init__(self, n_experts: int, percentile: float = 75.0):
        self.n_experts, self.percentile = n_experts, percentile
        self.load = defaultdict(lambda: torch.zeros(n_experts, dtype=torch.long))
        self.hits = defaultdict(int)
        self.total = defaultdict(int)
        self.overlap = defaultdict(list)
        self._prev: dict[int, torch.Tensor] = {}
        self._predicted: dict[int, torch.Tensor] = {}

    def predict(self, layer: int, ids: torch.Tensor) -> None:
        """Expert ids [T, k'] predicted for `layer` before its own router ran."""
        self._predicted[layer] = ids.detach().cpu()

    def observe(self, layer: int, ids: torch.Tensor) -> None:
        """Expert ids [T, k] the router of `layer` chose."""
        ids = ids.detach().cpu().long()
        self.load[layer] += torch.bincount(ids.flatten(), minlength=self.n_experts)
        pred = self._predicted.pop(layer, None)
        if pred is not None and pred.shape[0] == ids.shape[0]:
            hit = (ids.unsqueeze(-1) == pred.long().unsqueeze(1)).any(-1)
            self.hits[layer] += int(hit.sum())
            self.total[layer] += hit.numel()
        prev = self._prev.get(layer - 1)
        if prev is not None and prev.shape[0] == ids.shape[0]:
            same = (ids.unsqueeze(-1) == prev.unsqueeze(1)).any(-1).float().mean().item()
            self.overlap[layer].append(same)
        self._prev[layer] = ids

    def hit_rate(self, layer: int) -> float:
        return self.hits[layer] / self.total[layer] if self.total[layer] else 0.0

    def hot_experts(self, layer: int) -> list[int]:
        """Experts whose load is at or above the configured percentile of the layer's loads."""
        load = self.load[layer].float()
        thr = torch.quantile(load, self.percentile / 100.0)
        return [int(i) for i in torch.nonzero(load >= thr).flatten() if load[i] > 0]

    def summary(self) -> dict:
        return {int(l): {"tokens_routed": int(self.load[l].sum()), "hit_rate": round(self.hit_rate(l), 4),
                         "overlap_with_previous": round(sum(self.overlap[l]) / len(self.overlap[l]), 4) if self.overlap[l] else None,
                         "max_load_share": round(float(self.load[l].max()) / max(int(self.load[l].sum()), 1), 4)}
                for l in sorted(self.load)}
