"""The data plane between one trainer rank and the workers of a generation server: a process group that exists beside
the training job's own groups (the trainer is already rank r of its job; here it is rank 0 of a second, unrelated
world whose other ranks are the server's GPU workers).

The group is built from a ``TCPStore`` the trainer hosts and a process-group object constructed directly on it, so
neither side touches its default group. NCCL on GPUs (NVLink or network, whatever connects the trainer to the server),
gloo for CPU tests. Every wait is bounded: formation by the store timeout, each broadcast by ``wait(timeout)``.

Counterpart of the reference's vendored NCCL communicator and rendezvous listener
(halo/weight_sync/transport/pynccl.py:68-146, rendezvous.py) without a ctypes binding of the NCCL library: the
``torch.distributed`` group objects already expose a stateless constructor.
"""

from __future__ import annotations

import socket
from datetime import timedelta

import torch
import torch.distributed as dist

FORMATION_TIMEOUT_S = 120.0
CHUNK_TIMEOUT_S = 300.0


def free_port(host: str = "") -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]


def routable_address(toward: str | None = None) -> str:
    """The local address a peer at ``toward`` would see (no packet is sent: a UDP connect only picks the route)."""
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
            s.connect((toward or "10.255.255.255", 1))
            return s.getsockname()[0]
    except OSError:
        return "127.0.0.1"


class EngineGroup:
    """Rank ``rank`` of a ``world_size``-rank group rooted at ``host:port`` (rank 0 hosts the store)."""

    def __init__(self, host: str, port: int, rank: int, world_size: int, device=None, timeout_s: float = FORMATION_TIMEOUT_S,
                 backend: str | None = None):
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.backend = backend or ("nccl" if self.device.type == "cuda" else "gloo")
        timeout = timedelta(seconds=timeout_s)
        self.store = dist.TCPStore(host, port, world_size, is_master=(rank == 0), timeout=timeout, wait_for_workers=False)
        prefixed = dist.PrefixStore("halo_b200_engine_group", self.store)
        if self.backend == "nccl":
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = timeout
            self.pg = dist.ProcessGroupNCCL(prefixed, rank, world_size, opts)
        else:
            self.pg = dist.ProcessGroupGloo(prefixed, rank, world_size, timeout)
        self.closed = False

    def broadcast(self, tensor: torch.Tensor, src: int = 0, timeout_s: float = CHUNK_TIMEOUT_S) -> None:
        opts = dist.BroadcastOptions()
        opts.rootRank, opts.rootTensor = src, 0
        work = self.pg.broadcast([tensor], opts)
        if not work.wait(timedelta(seconds=timeout_s)):
            raise TimeoutError(f"a weight chunk of {tensor.numel() * tensor.element_size()} bytes did not reach the server "
                               f"within {timeout_s:.0f} s")
        if tensor.is_cuda:
            torch.cuda.current_stream(tensor.device).synchronize()

    def barrier(self, timeout_s: float = CHUNK_TIMEOUT_S) -> None:
        t = torch.zeros(1, device=self.device)
        opts = dist.AllreduceOptions()
        work = self.pg.allreduce([t], opts)
        if not work.wait(timedelta(seconds=timeout_s)):
            raise TimeoutError("the trainer-to-server group did not answer a barrier")

    def close(self) -> None:
        if not self.closed:
            self.closed = True
            self.pg = None
            self.store = None
