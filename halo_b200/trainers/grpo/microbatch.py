"""Token-budget micro-batch planning (halo/trainers/grpo/rounds/microbatch_plan.py:41-136) and the
rank-balanced deal of rows (halo/trainers/grpo/rounds/rank_balance.py:116-169).

Rows are packed into bins of at most ``budget`` tokens with first-fit-decreasing; every rank must run
the same number of micro-steps (each backward enters collectives), so the world agrees on the
maximum bin count and ranks with fewer bins get empty leading slots - leading, so that the last
backward of the window, which triggers the gradient reduction, is a real one."""

from __future__ import annotations


def first_fit_decreasing(lengths: list[int], budget: int) -> list[list[int]]:
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    bins: list[list[int]] = []
    loads: list[int] = []
    for i in order:
        n = lengths[i]
        if n > budget:
            raise ValueError(f"row {i} has {n} tokens, more than the micro-batch budget {budget}")
        for b in range(len(bins)):
            if loads[b] + n <= budget:
                bins[b].append(i)
                loads[b] += n
                break
        else:
            bins.append([i])
            loads.append(n)
    return bins


def balanced_partition(lengths: list[int], slots: int) -> list[list[int]]:
    """Longest-processing-time partition into exactly ``slots`` bins (some may stay empty)."""
    bins = [[] for _ in range(slots)]
    loads = [0] * slots
    for i in sorted(range(len(lengths)), key=lambda i: -lengths[i]):
        b = min(range(slots), key=lambda j: loads[j])
        bins[b].append(i)
        loads[b] += lengths[i]
    return bins


def plan_microbatches(lengths: list[int], budget: int, world_max_bins=None) -> list[list[int]]:
    """This rank's bins, padded with leading empty bins up to the world's maximum bin count.
    ``world_max_bins``: callable(int) -> int performing the MAX reduction over ranks (None = single rank)."""
    bins = first_fit_decreasing(lengths, budget) if lengths else []
    if not bins:
        bins = [[]]
    n = world_max_bins(len(bins)) if world_max_bins is not None else len(bins)
    if n > len(bins):
        if len(lengths) >= n:
            bins = [b for b in balanced_partition(lengths, n)]
            bins.sort(key=len)
        else:
            bins = [[] for _ in range(n - len(bins))] + bins
    return bins


def deal_rows_across_ranks(lengths: list[int], world: int) -> list[list[int]]:
    """Rows dealt to ranks by attended tokens (LPT), keeping row counts equal up to one."""
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    per = [[] for _ in range(world)]
    loads = [0] * world
    cap = -(-len(lengths) // world)
    for i in order:
        open_ranks = [r for r in range(world) if len(per[r]) < cap]
        r = min(open_ranks, key=lambda j: loads[j])
        per[r].append(i)
        loads[r] += lengths[i]
    return per
