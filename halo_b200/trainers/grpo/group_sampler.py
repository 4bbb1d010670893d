"""Which stored rollouts a data-parallel rank trains on in each round of offline GRPO.

Rows are ordered by group (the generations of one prompt), the groups are cut contiguously over the data-parallel ranks,
and every rank walks its own groups in an order shuffled by a seed that does NOT depend on the rank and changes with the
epoch. A rank always holds whole groups: the trainer forms group advantages from the rewards it is handed, so a group
must not straddle two ranks (the reference precomputes advantages per row and lets a group straddle; the cut here falls
on the next group boundary instead). Every rank gets the same number of groups - the remainder of the division is
dropped - so all ranks run the same number of rounds and nobody waits in a collective for a rank that has finished.
Ranks that share one data-parallel slice (tensor-, context- or pipeline-parallel siblings) pass the same
``(rank, world)`` and therefore iterate identical rows in identical order.

(The role of halo/trainers/grpo/offline/group_sampler.py:17-62 and its batch-count equalisation, :113-146.)"""

from __future__ import annotations

import random
from collections import OrderedDict


class GroupSampler:
    def __init__(self, group_ids, rank: int = 0, world: int = 1, groups_per_round: int = 64, shuffle: bool = True, seed: int = 0):
        if not 0 <= rank < world:
            raise ValueError(f"rank {rank} is outside a data-parallel width of {world}")
        groups: OrderedDict = OrderedDict()
        for i, gid in enumerate(group_ids):
            groups.setdefault(gid, []).append(i)
        ordered = list(groups.values())                       # first-seen order of the groups, rows of a group together
        per_rank = len(ordered) // world
        if per_rank == 0:
            raise ValueError(f"{len(ordered)} groups cannot be cut over {world} data-parallel ranks: a rank would train on "
                             "nothing while its peers wait for it")
        self.n_groups_total, self.dropped_groups = len(ordered), len(ordered) - per_rank * world
        self.groups = ordered[rank * per_rank:(rank + 1) * per_rank]
        self.groups_per_round = max(1, int(groups_per_round))
        self.shuffle, self.seed, self.epoch = shuffle, int(seed), 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = int(epoch)

    @property
    def rounds_per_epoch(self) -> int:
        return (len(self.groups) + self.groups_per_round - 1) // self.groups_per_round

    def order(self, epoch: int | None = None) -> list[int]:
        """Positions of this rank's groups in the order of ``epoch`` (the same permutation on every rank)."""
        idx = list(range(len(self.groups)))
        if self.shuffle:
            random.Random(self.seed + (self.epoch if epoch is None else epoch)).shuffle(idx)
        return idx

    def round_rows(self, round_index: int, epochs: float = 1.0) -> list[int] | None:
        """Row indices of round ``round_index`` counted from the start of training (groups whole and consecutive), or
        None once ``epochs`` passes over this rank's groups are done."""
        per = self.rounds_per_epoch
        if round_index >= int(round(per * epochs)):
            return None
        epoch, r = divmod(round_index, per)
        order = self.order(epoch)[r * self.groups_per_round:(r + 1) * self.groups_per_round]
        return [i for g in order for i in self.groups[g]]

    def __len__(self) -> int:
        return sum(len(g) for g in self.groups)
