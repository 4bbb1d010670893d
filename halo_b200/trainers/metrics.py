"""Rank-local metrics staged on the device and folded over the world with ONE collective per log
(halo/trainers/metrics/world_metrics.py:219-396).

``add_sum`` / ``add_mean`` / ``add_max`` / ``add_fraction`` stage values without a host sync; ``reduce`` packs every
staged column into one tensor, all-reduces it once (sums and counts with SUM; maxima ride along negated-min style in
a second segment reduced with MAX) and returns plain floats."""

from __future__ import annotations

import torch
import torch.distributed as dist


class WorldMetrics:
    def __init__(self, device="cpu", group=None):
        self.device, self.group = torch.device(device), group
        self._sums: dict[str, torch.Tensor] = {}
        self._means: dict[str, list] = {}
        self._maxes: dict[str, torch.Tensor] = {}

    def _t(self, v):
        return v.detach().to(self.device, torch.float64).reshape(()) if isinstance(v, torch.Tensor) else \
            torch.tensor(float(v), dtype=torch.float64, device=self.device)

    def add_sum(self, name: str, value) -> None:
        self._sums[name] = self._sums.get(name, 0) + self._t(value)

    def add_mean(self, name: str, value_sum, count) -> None:
        """Mean of per-token (or per-sample) values: stage the numerator and the denominator."""
        cur = self._means.get(name)
        num, den = self._t(value_sum), self._t(count)
        self._means[name] = [num, den] if cur is None else [cur[0] + num, cur[1] + den]

    def add_fraction(self, name: str, hits, total) -> None:
        self.add_mean(name, hits, total)

    def add_max(self, name: str, value) -> None:
        v = self._t(value)
        self._maxes[name] = v if name not in self._maxes else torch.maximum(self._maxes[name], v)

    def reduce(self) -> dict[str, float]:
        names_s, names_m, names_x = sorted(self._sums), sorted(self._means), sorted(self._maxes)
        cols = [self._sums[n] for n in names_s] + [x for n in names_m for x in self._means[n]]
        live = dist.is_available() and dist.is_initialized()
        out: dict[str, float] = {}
        if cols:
            packed = torch.stack(cols)
            if live:
                dist.all_reduce(packed, group=self.group)               # the one collective for sums and means
            vals = packed.tolist()
            for i, n in enumerate(names_s):
                out[n] = vals[i]
            base = len(names_s)
            for j, n in enumerate(names_m):
                num, den = vals[base + 2 * j], vals[base + 2 * j + 1]
                out[n] = num / den if den else 0.0
        if names_x:
            packed = torch.stack([self._maxes[n] for n in names_x])
            if live:
                dist.all_reduce(packed, op=dist.ReduceOp.MAX, group=self.group)
            for n, v in zip(names_x, packed.tolist()):
                out[n] = v
        self._sums.clear()
        self._means.clear()
        self._maxes.clear()
        return out
