"""Summarise a ``torch.profiler`` Chrome trace:  python -m halo_b200.diagnostics.trace_report trace.json [--top 25]

Device time per kernel (launches, total, mean, share), grouped into families (GEMM, attention, expert rows, norms and
other element-wise kernels, optimizer, collectives / peer copies, library kernels), plus how much of the profiled span
the device was busy and how much of the busy time overlapped between streams. Reads plain or gzip-compressed traces.
The role of the reference's trace report (scripts/profiling/trace_report.py)."""

from __future__ import annotations

import argparse
import gzip
import json
import re
import sys
from collections import defaultdict

FAMILIES = [
    ("gemm", re.compile(r"gemm_bf16|halo_gemm|cutlass|cublas|gemm|sgemm|ampere_|sm90_|sm100_", re.I)),
    ("attention", re.compile(r"attn|attention|flash", re.I)),
    ("expert rows", re.compile(r"dispatch_rows|combine_rows|route_|router_topk|swiglu_bwd_weighted|zero_pad_rows|gather_slot", re.I)),
    ("optimizer", re.compile(r"adamw|grad_sq|clip|muon", re.I)),
    ("collectives", re.compile(r"nccl|peer_pull|reduce_scatter|all_gather|allreduce|broadcast_bytes", re.I)),
    ("element-wise", re.compile(r"rmsnorm|rope|swiglu|cross_entropy|logprob|stream_|sinkhorn|fake_quant|elementwise|vectorized", re.I)),
]


def family_of(name: str) -> str:
    for fam, rx in FAMILIES:
        if rx.search(name):
            return fam
    return "other"


def load_events(path: str) -> list[dict]:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        data = json.load(f)
    events = data["traceEvents"] if isinstance(data, dict) else data
    return [e for e in events if e.get("ph") == "X" and e.get("cat", "").lower() in ("kernel", "gpu_memcpy", "gpu_memset")]


def busy_time(intervals: list[tuple[float, float]]) -> float:
    total, end = 0.0, float("-inf")
    for lo, hi in sorted(intervals):
        if hi <= end:
            continue
        total += hi - max(lo, end)
        end = hi
    return total


def summarise(events: list[dict], top: int = 25) -> dict:
    per = defaultdict(lambda: [0, 0.0])
    fam = defaultdict(float)
    by_stream = defaultdict(list)
    for e in events:
        name, dur = e["name"], float(e["dur"])
        per[name][0] += 1
        per[name][1] += dur
        fam[family_of(name)] += dur
        by_stream[(e.get("pid"), e.get("tid"))].append((float(e["ts"]), float(e["ts"]) + dur))
    total = sum(v[1] for v in per.values())
    everything = [iv for ivs in by_stream.values() for iv in ivs]
    span = (max(hi for _, hi in everything) - min(lo for lo, _ in everything)) if everything else 0.0
    busy = busy_time(everything)
    kernels = sorted(({"name": n, "launches": c, "total_us": t, "mean_us": t / c, "share": t / total if total else 0.0}
                      for n, (c, t) in per.items()), key=lambda r: -r["total_us"])
    return {"kernels": kernels[:top], "families": dict(sorted(fam.items(), key=lambda kv: -kv[1])), "device_time_us": total,
            "span_us": span, "busy_us": busy, "busy_fraction": busy / span if span else 0.0,
            "overlap_us": total - busy, "launches": sum(v[0] for v in per.values())}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("trace")
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    rep = summarise(load_events(args.trace), args.top)
    if args.json:
        print(json.dumps(rep))
        return 0
    print(f"{rep['launches']} launches, {rep['device_time_us'] / 1e3:.2f} ms of device time over a span of {rep['span_us'] / 1e3:.2f} ms "
          f"(busy {rep['busy_fraction']:.0%}, {rep['overlap_us'] / 1e3:.2f} ms overlapped between streams)")
    for name, t in rep["families"].items():
        print(f"  {name:14s} {t / 1e3:10.3f} ms  {t / rep['device_time_us']:6.1%}")
    print(f"{'kernel':70s} {'launches':>8s} {'total ms':>10s} {'mean us':>9s} {'share':>6s}")
    for k in rep["kernels"]:
        print(f"{k['name'][:70]:70s} {k['launches']:8d} {k['total_us'] / 1e3:10.3f} {k['mean_us']:9.1f} {k['share']:6.1%}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
