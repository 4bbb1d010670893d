"""Spawn N CPU ranks with a gloo process group for multi-rank tests (bounded: a hung rank is killed)."""

from __future__ import annotations

import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, worker, args, errq):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "LOCAL_WORLD_SIZE": str(world), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                       "OMP_NUM_THREADS": "1"})
    import torch
    import torch.distributed as dist

    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        worker(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except BaseException:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
        raise


def run_gloo_ranks(worker, nprocs: int = 2, args: tuple = (), timeout: float = 240.0):
    """``worker(rank, world, *args)`` runs in ``nprocs`` spawned processes; raises if any fails or hangs."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, nprocs, port, worker, args, errq), daemon=True) for r in range(nprocs)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    if errors:
        raise AssertionError("\n".join(f"--- rank {r} ---\n{tb}" for r, tb in errors))
    if hung:
        raise AssertionError(f"{len(hung)} rank(s) did not finish within {timeout} s")
    bad = [p.exitcode for p in procs if p.exitcode != 0]
    if bad:
        raise AssertionError(f"ranks exited with codes {bad}")
