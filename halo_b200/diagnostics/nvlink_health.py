"""Peer-to-peer health of one box (halo scripts/profiling/nvlink_health.py): for every ordered GPU pair, can the
destination's memory be accessed from the source and how fast does a 256 MiB copy go. Run on a machine with GPUs:

    python -m halo_b200.diagnostics.nvlink_health

Copies are plain ``cudaMemcpyAsync`` device-to-device transfers timed with CUDA events after a warm-up copy."""

from __future__ import annotations

import json
import sys

import torch


def pair_bandwidth(src: int, dst: int, nbytes: int = 256 << 20, iters: int = 5) -> float:
    a = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{src}")
    b = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{dst}")
    with torch.cuda.device(src):
        b.copy_(a)
        torch.cuda.synchronize(src)
        best = 0.0
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            b.copy_(a, non_blocking=True)
            e1.record()
            torch.cuda.synchronize(src)
            best = max(best, nbytes / (e0.elapsed_time(e1) * 1e6))
    return best      # GB/s


def main() -> int:
    n = torch.cuda.device_count()
    if n < 2:
        print("fewer than two GPUs: nothing to measure")
        return 0
    report = {"gpus": n, "peer_access": {}, "gb_per_s": {}}
    worst = None
    for s in range(n):
        for d in range(n):
            if s == d:
                continue
            ok = torch.cuda.can_device_access_peer(s, d)
            report["peer_access"][f"{s}->{d}"] = ok
            if ok:
                bw = pair_bandwidth(s, d)
                report["gb_per_s"][f"{s}->{d}"] = round(bw, 1)
                worst = bw if worst is None else min(worst, bw)
    report["slowest_pair_gb_per_s"] = round(worst, 1) if worst is not None else None
    json.dump(report, sys.stdout, indent=1)
    print()
    return 0 if all(report["peer_access"].values()) else 1


if __name__ == "__main__":
    sys.exit(main())
