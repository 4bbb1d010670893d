"""``ParallelismConfig``: the sizes of the five model-sharding axes (EP, ETP, TP, CP, PP), the data
parallel width that is left, this rank's coordinates, and the group memberships derived from them.

Pure arithmetic: constructing a config touches no process group, so the same object describes
rank 3 of 8 on a GPU box or rank 731 of 1,024 in a CPU test. ``data_parallel_size`` is
``stage_world / max(tp, cp, etp)`` and EP is orthogonal to it, as in the reference
(halo/distributed/parallelism_config.py:33-483, rules at halo/distributed/parallelism_rules.py).
The user-facing field names are kept so existing YAML recipes carry over.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

from halo_b200.config_validation import ConfigError

from . import layout as L
from .rules import reject_invalid_composition, reject_unsupported_axes

AXIS_FIELDS = (
    ("pp", "pipeline_parallel_size", "pp_size"),
    ("ep", "expert_parallel_size", "ep_size"),
    ("etp", "expert_tensor_parallel_size", "expert_tp_size"),
    ("tp", "tensor_parallel_size", "tp_size"),
    ("cp", "context_parallel_size", "cp_size"),
)


@dataclass
class ParallelismConfig:
    world_size: int = 0          # 0 = WORLD_SIZE
    global_rank: int = -1        # -1 = RANK
    gpus_per_node: int = 0       # 0 = LOCAL_WORLD_SIZE, else the world
    nvlink_domain_size: int = 0  # 0 = NVLINK_DOMAIN_SIZE, else gpus_per_node

    ep_size: int = 1
    expert_tp_size: int = 1
    tp_size: int = 1
    cp_size: int = 1
    pp_size: int = 1
    pp_schedule: str = "1f1b"          # "1f1b" | "gpipe"
    pp_microbatches: int = 0            # 0 = gradient_accumulation_steps
    pp_split: list[int] | None = None   # decoder layers per stage; None = head-weighted default
    ep_scope: str = "auto"              # "auto" | "node" | "global"
    ep_buffer_backend: str = "auto"     # kept for recipe compatibility: "auto" | "symmetric" | "nccl"

    fp32_router: bool = False
    fp32_experts: bool = False
    fp32_non_ep_params: bool = False
    fp32_grad_reduce: bool = False
    bf16_optimizer: bool | None = None
    use_grouped_gemm: bool = True
    fsdp_reshard_after_forward: bool = False
    fsdp_reshard_after_backward: bool = True
    fsdp_defer_grad_sync: bool = False
    fsdp_shard_ep1_experts: bool = True
    use_hsdp: bool = False
    max_concurrent_loading: int | None = None
    ep_lazy_loading: bool = True
    init_from_scratch: bool = False

    # derived
    ep_group_size: int = field(default=0, init=False)
    stage_world_size: int = field(default=0, init=False)
    data_parallel_size: int = field(default=0, init=False)
    num_nodes: int = field(default=0, init=False)
    num_nvlink_domains: int = field(default=0, init=False)
    pp_rank: int = field(default=0, init=False)
    stage_base_rank: int = field(default=0, init=False)
    stage_local_rank: int = field(default=0, init=False)

    def __post_init__(self):
        self._resolve_world()
        self._validate_fields()
        reject_unsupported_axes(self)
        self._resolve_topology()
        reject_invalid_composition(self)

    # ---- resolution ------------------------------------------------------------------------
    def _resolve_world(self) -> None:
        explicit_world = self.world_size > 0     # a subset of the job (the trainer ranks of a split job)
        if self.world_size <= 0:
            self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        if self.global_rank < 0:
            self.global_rank = int(os.environ.get("RANK", "0"))
        if self.gpus_per_node <= 0:
            self.gpus_per_node = int(os.environ.get("LOCAL_WORLD_SIZE", "0")) or self.world_size
            if explicit_world and self.world_size < self.gpus_per_node:
                self.gpus_per_node = self.world_size
        if self.nvlink_domain_size <= 0:
            self.nvlink_domain_size = int(os.environ.get("NVLINK_DOMAIN_SIZE", "0") or 0) or self.gpus_per_node
        if not 0 <= self.global_rank < self.world_size:
            raise ConfigError(f"rank {self.global_rank} is outside a world of {self.world_size}")

    def _validate_fields(self) -> None:
        for _, flag, attr in AXIS_FIELDS:
            v = getattr(self, attr)
            if not isinstance(v, int) or v < 1:
                raise ConfigError(f"{flag} must be an integer >= 1, got {v!r}")
        if self.pp_schedule not in ("1f1b", "gpipe"):
            raise ConfigError(f"pipeline_schedule must be '1f1b' or 'gpipe', got {self.pp_schedule!r}")
        if self.ep_scope not in ("auto", "node", "global"):
            raise ConfigError(f"ep_scope must be 'auto', 'node' or 'global', got {self.ep_scope!r}")
        if self.ep_buffer_backend not in ("auto", "symmetric", "nccl", "elastic", "legacy"):
            raise ConfigError(f"ep_buffer_backend {self.ep_buffer_backend!r} is not known")
        if self.world_size % self.gpus_per_node:
            raise ConfigError(f"world_size ({self.world_size}) is not a multiple of gpus_per_node ({self.gpus_per_node})")

    def _resolve_topology(self) -> None:
        if self.world_size % self.pp_size:
            raise ConfigError(
                f"world_size ({self.world_size}) must be divisible by pipeline_parallel_size ({self.pp_size}): "
                f"pipeline stages are equal contiguous rank blocks.")
        self.stage_world_size = self.world_size // self.pp_size
        self.ep_group_size = self.ep_size * self.expert_tp_size
        self.nvlink_domain_size = min(self.nvlink_domain_size, self.stage_world_size) or 1
        if self.ep_scope == "auto":
            self.ep_scope = "node" if self.ep_group_size <= self.nvlink_domain_size else "global"
        elif self.ep_group_size == 1:
            self.ep_scope = "node"
        self.num_nodes = max(1, self.world_size // self.gpus_per_node)
        self.num_nvlink_domains = max(1, self.stage_world_size // self.nvlink_domain_size)
        widest = max(self.tp_size, self.cp_size, self.expert_tp_size)
        if self.stage_world_size % widest:
            raise ConfigError(
                f"the stage width ({self.stage_world_size}) is not divisible by the widest of tensor / context / "
                f"expert-tensor parallel sizes ({widest})")
        self.data_parallel_size = self.stage_world_size // widest
        self.pp_rank = self.global_rank // self.stage_world_size
        self.stage_base_rank = self.pp_rank * self.stage_world_size
        self.stage_local_rank = self.global_rank % self.stage_world_size

    # ---- facts -----------------------------------------------------------------------------
    @property
    def active_axes(self) -> frozenset[str]:
        return frozenset(name for name, _, attr in AXIS_FIELDS if getattr(self, attr) > 1)

    @property
    def has_ep_group(self) -> bool:
        return self.ep_group_size > 1

    @property
    def experts_dp_sharded(self) -> bool:
        """With no expert-distribution group the experts are ordinary data-parallel parameters."""
        return self.fsdp_shard_ep1_experts and self.ep_group_size == 1

    @property
    def non_dp_replication_factor(self) -> int:
        """Ranks that see the same tokens (token counters are divided by it)."""
        return max(self.tp_size, self.cp_size, self.expert_tp_size)

    @property
    def reduces_in_fp32(self) -> bool:
        return self.fp32_grad_reduce or self.fp32_non_ep_params

    def pp_microbatch_count(self, gradient_accumulation_steps: int) -> int:
        n = self.pp_microbatches or gradient_accumulation_steps
        return max(n, self.pp_size) if self.pp_schedule == "1f1b" else n

    # ---- group memberships (stage-local rank space, then shifted to global ranks) ---------------
    @property
    def ep_layout(self):
        return L.make_layout(self.stage_world_size, self.ep_group_size, self.nvlink_domain_size,
                             domain_local=self.ep_scope == "node")

    def _globalise(self, ranks: list[int]) -> list[int]:
        return [self.stage_base_rank + r for r in ranks]

    @property
    def ep_position(self) -> int:
        return self.ep_layout.locate(self.stage_local_rank)[0]

    @property
    def dispatch_ep_rank(self) -> int:
        return self.ep_layout.split_expert_tp(self.ep_position, self.ep_size, self.expert_tp_size)[0]

    @property
    def expert_tp_rank(self) -> int:
        return self.ep_layout.split_expert_tp(self.ep_position, self.ep_size, self.expert_tp_size)[1]

    def ep_group_ranks(self) -> list[int]:
        _, g = self.ep_layout.locate(self.stage_local_rank)
        return self._globalise(self.ep_layout.group_ranks(g))

    def dispatch_group_ranks(self) -> list[int]:
        """The ranks that exchange tokens with this one: same expert-TP rank, every dispatch rank."""
        lay = self.ep_layout
        _, g = lay.locate(self.stage_local_rank)
        members = lay.group_ranks(g)
        mine = self.expert_tp_rank
        keep = [r for pos, r in enumerate(members)
                if lay.split_expert_tp(pos, self.ep_size, self.expert_tp_size)[1] == mine]
        return self._globalise(keep)

    def expert_tp_group_ranks(self) -> list[int]:
        lay = self.ep_layout
        _, g = lay.locate(self.stage_local_rank)
        members = lay.group_ranks(g)
        mine = self.dispatch_ep_rank
        keep = [r for pos, r in enumerate(members)
                if lay.split_expert_tp(pos, self.ep_size, self.expert_tp_size)[0] == mine]
        return self._globalise(keep)

    def expert_replica_ranks(self) -> list[int]:
        """Ranks of this stage holding the same expert shard (their expert gradients are summed)."""
        return self._globalise(self.ep_layout.replica_ranks(self.ep_position))

    def tp_group_ranks(self) -> list[int]:
        base = self.stage_local_rank // self.tp_size * self.tp_size
        return self._globalise(list(range(base, base + self.tp_size)))

    def cp_group_ranks(self) -> list[int]:
        base = self.stage_local_rank // self.cp_size * self.cp_size
        return self._globalise(list(range(base, base + self.cp_size)))

    def dp_group_ranks(self) -> list[int]:
        """Ranks of this stage that hold different batches at the same tensor/context position."""
        w = self.non_dp_replication_factor
        pos = self.stage_local_rank % w
        return self._globalise([g * w + pos for g in range(self.stage_world_size // w)])

    def stage_ranks(self) -> list[int]:
        return self._globalise(list(range(self.stage_world_size)))

    def pp_chain_ranks(self) -> list[int]:
        return [s * self.stage_world_size + self.stage_local_rank for s in range(self.pp_size)]

    @property
    def data_parallel_rank(self) -> int:
        return self.stage_local_rank // self.non_dp_replication_factor

    def all_groups(self, kind: str) -> list[list[int]]:
        """Every group of one kind in the job, in the creation order all ranks share."""
        seen, out = set(), []
        for r in range(self.world_size):
            other = self.for_rank(r)
            ranks = tuple(getattr(other, f"{kind}_ranks")() if not kind.endswith("_ranks") else getattr(other, kind)())
            if ranks not in seen:
                seen.add(ranks)
                out.append(list(ranks))
        return out

    def for_rank(self, rank: int) -> "ParallelismConfig":
        """The same layout seen from another rank (no collectives, no environment reads)."""
        kw = {f: getattr(self, f) for f in (
            "world_size", "gpus_per_node", "nvlink_domain_size", "ep_size", "expert_tp_size", "tp_size", "cp_size",
            "pp_size", "pp_schedule", "pp_microbatches", "pp_split", "ep_buffer_backend", "fp32_router",
            "fp32_experts", "fp32_non_ep_params", "fp32_grad_reduce", "bf16_optimizer", "use_grouped_gemm",
            "fsdp_reshard_after_forward", "fsdp_reshard_after_backward", "fsdp_defer_grad_sync",
            "fsdp_shard_ep1_experts", "use_hsdp", "max_concurrent_loading", "ep_lazy_loading", "init_from_scratch")}
        kw["ep_scope"] = self.ep_scope
        kw["global_rank"] = rank
        return ParallelismConfig(**kw)

    def fingerprint(self) -> dict:
        """What must match for optimizer shards to be resumed exactly."""
        return {"world_size": self.world_size, "pp": self.pp_size, "ep": self.ep_size, "etp": self.expert_tp_size,
                "tp": self.tp_size, "cp": self.cp_size, "pp_split": list(self.pp_split) if self.pp_split else None}
