"""Context-parallel attention against the single-GPU flash kernels: forward and forward + backward of one packed row cut
over the ranks, timed on the device (CUDA events, max over ranks, median), for one long document and for chat-length
documents.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/context_parallel.py [out.json]

The target is (single-GPU time) / N: keys and values are read from their owners inside the kernels, so no transfer sits
on the critical path, and the paired early / late pieces give every rank the same causal work. `--tokens=T` sets the row
length (default 65536), `--contiguous` times contiguous chunks instead of paired pieces, `--direct-reads` lets the kernels
read every foreign tile from its owner instead of from the local mirror.
"""

from __future__ import annotations

import json
import os
import statistics
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters=5, warmup=2):
    out = []
    for i in range(warmup + iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if i >= warmup:
            out.append(float(ms.item()))
    return statistics.median(out)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from halo_b200.ops import _lib
    from halo_b200.ops import attention as attn_ops
    from halo_b200.parallel.context_parallel import TILE, CPExchange, build_cp_plan, cp_attention, make_layout

    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    total = next((int(a.split("=", 1)[1]) for a in sys.argv[1:] if a.startswith("--tokens=")), 65536)
    balance = "--contiguous" not in sys.argv
    Hq, Hkv, D = 32, 4, 128
    rng = np.random.default_rng(1)
    lens, left = [], total
    while left > 0:
        n = int(min(left, np.clip(rng.lognormal(np.log(990), 0.6), 64, 4579)))
        lens.append(n)
        left -= n
    cases = {"one document": np.array([0, total]), "chat-length documents": np.concatenate([[0], np.cumsum(lens)])}
    direct = "--direct-reads" in sys.argv
    ex = CPExchange(dist.group.WORLD, dev, total // world + 4 * TILE, total + TILE, 2 * Hkv * D, direct_reads=direct)
    rows = []
    for name, cu in cases.items():
        g = torch.Generator(device=dev).manual_seed(3)
        q = (torch.randn(total, Hq * D, device=dev, generator=g) * 0.5).bfloat16()
        k = (torch.randn(total, Hkv * D, device=dev, generator=g) * 0.5).bfloat16()
        v = (torch.randn(total, Hkv * D, device=dev, generator=g) * 0.5).bfloat16()
        do = (torch.randn(total, Hq * D, device=dev, generator=g) * 0.5).bfloat16()
        plan1 = attn_ops.build_plan(cu, dev)
        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))

        def single_fwd():
            with torch.no_grad():
                attn_ops.flash_attention(qf, kf, vf, plan1, Hq, Hkv)

        def single_both():
            qf.grad = kf.grad = vf.grad = None
            attn_ops.flash_attention(qf, kf, vf, plan1, Hq, Hkv).backward(do)

        lay = make_layout(cu, rank, world, balance)
        idx = torch.from_numpy(lay.local_index()).to(dev)
        plan = build_cp_plan(lay, dev)
        ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
        dol = do[idx].contiguous()

        def cp_fwd():
            with torch.no_grad():
                cp_attention(ql, kl, vl, lay, plan, dist.group.WORLD, ex, Hq, Hkv)

        def cp_both():
            ql.grad = kl.grad = vl.grad = None
            cp_attention(ql, kl, vl, lay, plan, dist.group.WORLD, ex, Hq, Hkv).backward(dol)

        s_f, s_b = timed(single_fwd), timed(single_both)
        c_f, c_b = timed(cp_fwd), timed(cp_both)
        _lib.raise_on_status(dev)
        rows.append({"case": name, "tokens": total, "ranks": world, "pieces": "paired" if balance else "contiguous",
                     "keys_and_values": "tiles read from their owners" if direct else "rows fetched once into a local mirror",
                     "single_gpu_fwd_ms": round(s_f, 3), "single_gpu_fwd_bwd_ms": round(s_b, 3),
                     "cp_fwd_ms": round(c_f, 3), "cp_fwd_bwd_ms": round(c_b, 3),
                     "fwd_vs_single_over_ranks": round(c_f / (s_f / world), 3),
                     "fwd_bwd_vs_single_over_ranks": round(c_b / (s_b / world), 3)})
        if rank == 0:
            print(json.dumps(rows[-1]), flush=True)
    if rank == 0 and args:
        os.makedirs(os.path.dirname(args[0]) or ".", exist_ok=True)
        json.dump(rows, open(args[0], "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
