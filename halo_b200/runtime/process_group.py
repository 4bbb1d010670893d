"""Default process-group set-up: one process per GPU, NCCL bound to ``cuda:LOCAL_RANK`` with
``device_id`` so later sub-groups come from ``split_group``, and one timeout for every group
(the role of halo/runtime/process_group.py:76-114). CPU runs (tests, gloo ranks) use gloo."""

from __future__ import annotations

import logging
import os

import torch
import torch.distributed as dist

from halo_b200 import env
from halo_b200.runtime.ranks import get_local_rank

log = logging.getLogger(__name__)


def init_distributed(backend: str | None = None) -> torch.device:
    """Initialise the default group when the launcher set WORLD_SIZE > 1; returns this rank's device."""
    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda", get_local_rank()) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if use_cuda else "gloo")
        kwargs = {"timeout": env.nccl_timeout()}
        if backend == "nccl":
            kwargs["device_id"] = device
        dist.init_process_group(backend, **kwargs)
        log.info("process group up: backend=%s world=%d rank=%d", backend, world, dist.get_rank())
    return device


def destroy_distributed() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def default_timeout():
    return env.nccl_timeout()
