"""Rank layouts: which ranks of a pipeline stage form which group (pure arithmetic, no process
groups), for 1 to thousands of ranks.

``BlockLayout`` tiles every NVLink domain with contiguous blocks; ``StridedLayout`` gives each
group one contiguous block in *every* domain (a group that spans domains with an equal share in
each). Same grouping rules as the reference's ``NodeLocalLayout`` / ``CrossNodeLayout``
(halo/distributed/group_layout.py:9-106); on one 8-GPU NVSwitch box only ``BlockLayout`` occurs.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class BlockLayout:
    world_size: int
    group_size: int
    domain_size: int

    def __post_init__(self):
        if self.group_size < 1 or self.domain_size % self.group_size or self.world_size % self.domain_size:
            raise ValueError(
                f"group size {self.group_size} must divide the NVLink domain ({self.domain_size}), which must "
                f"divide the stage width ({self.world_size})")

    @property
    def groups_per_domain(self) -> int:
        return self.domain_size // self.group_size

    @property
    def num_groups(self) -> int:
        return self.world_size // self.group_size

    def locate(self, rank: int) -> tuple[int, int]:
        """(position inside its group, group index) of ``rank``."""
        return rank % self.group_size, rank // self.group_size

    def group_ranks(self, group: int) -> list[int]:
        return list(range(group * self.group_size, (group + 1) * self.group_size))

    def replica_ranks(self, position: int) -> list[int]:
        """The ranks sitting at ``position`` of every group (holders of the same shard)."""
        return [g * self.group_size + position for g in range(self.num_groups)]

    def split_expert_tp(self, position: int, ep_size: int, etp_size: int) -> tuple[int, int]:
        """(dispatch rank, expert-TP rank): an EP group is ``etp_size`` contiguous dispatch chunks."""
        return position % ep_size, position // ep_size


@dataclass(frozen=True)
class StridedLayout:
    world_size: int
    group_size: int
    domain_size: int

    def __post_init__(self):
        if self.domain_size < 1 or self.world_size % self.domain_size:
            raise ValueError(f"stage width {self.world_size} is not a multiple of the NVLink domain {self.domain_size}")
        nd = self.world_size // self.domain_size
        if self.group_size % nd:
            raise ValueError(
                f"a cross-domain group of {self.group_size} ranks must take an equal share of each of the {nd} "
                f"domains; use a group as wide as the stage ({self.world_size}) or a domain-local group")
        if self.domain_size % (self.group_size // nd):
            raise ValueError(
                f"{self.group_size // nd} members per domain do not tile a domain of {self.domain_size}")

    @property
    def num_domains(self) -> int:
        return self.world_size // self.domain_size

    @property
    def per_domain(self) -> int:
        return self.group_size // self.num_domains

    @property
    def num_groups(self) -> int:
        return self.domain_size // self.per_domain

    def locate(self, rank: int) -> tuple[int, int]:
        domain, pos = divmod(rank, self.domain_size)
        return domain * self.per_domain + pos % self.per_domain, pos // self.per_domain

    def group_ranks(self, group: int) -> list[int]:
        return [d * self.domain_size + group * self.per_domain + i
                for d in range(self.num_domains) for i in range(self.per_domain)]

    def replica_ranks(self, position: int) -> list[int]:
        domain, i = divmod(position, self.per_domain)
        return [domain * self.domain_size + g * self.per_domain + i for g in range(self.num_groups)]

    def split_expert_tp(self, position: int, ep_size: int, etp_size: int) -> tuple[int, int]:
        return position // etp_size, position % etp_size


def make_layout(world_size: int, group_size: int, domain_size: int, domain_local: bool):
    return (BlockLayout if domain_local else StridedLayout)(world_size, group_size, domain_size)


def contiguous_groups(world_size: int, group_size: int) -> list[list[int]]:
    """TP / CP / expert-TP style groups: consecutive ranks."""
    if world_size % group_size:
        raise ValueError(f"{group_size} does not divide {world_size}")
    return [list(range(s, s + group_size)) for s in range(0, world_size, group_size)]


def strided_groups(world_size: int, group_size: int) -> list[list[int]]:
    """The complementary groups of ``contiguous_groups``: ranks with the same position."""
    n = world_size // group_size
    return [[g * group_size + p for g in range(n)] for p in range(group_size)]
