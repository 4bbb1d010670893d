"""Rank and world getters that work before ``init_process_group`` (torchrun or SLURM variables),
node arithmetic and a rank tag for file names (the role of halo/runtime/ranks.py)."""

from __future__ import annotations

import os


def _env_int(*names: str, default: int) -> int:
    for n in names:
        v = os.environ.get(n)
        if v is not None and v.strip():
            try:
                return int(v)
            except ValueError:
                continue
    return default


def get_global_rank() -> int:
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:  # pragma: no cover
        pass
    return _env_int("RANK", "SLURM_PROCID", default=0)


def get_world_size() -> int:
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_world_size()
    except Exception:  # pragma: no cover
        pass
    return _env_int("WORLD_SIZE", "SLURM_NTASKS", default=1)


def get_local_rank() -> int:
    return _env_int("LOCAL_RANK", "SLURM_LOCALID", default=0)


def get_local_world_size() -> int:
    return _env_int("LOCAL_WORLD_SIZE", "SLURM_NTASKS_PER_NODE", default=get_world_size())


def get_node_rank() -> int:
    return get_global_rank() // max(1, get_local_world_size())


def get_num_nodes() -> int:
    return max(1, get_world_size() // max(1, get_local_world_size()))


def is_global_main_process() -> bool:
    return get_global_rank() == 0


def is_local_main_process() -> bool:
    return get_local_rank() == 0


def is_distributed() -> bool:
    return get_world_size() > 1


def rank_tag() -> str:
    return f"rank{get_global_rank():05d}"
