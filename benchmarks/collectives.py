"""Multi-GPU kernel benchmarks: the kernels that compute and move data over NVLink in one launch, each against its
roofline (the slower of FLOPs / measured sustained GEMM rate and NVLink bytes / 900 GB/s per direction per GPU) and
against the library baseline (NCCL collective + separate kernel).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/collectives.py

Timing: CUDA events on the launching stream after warm-up, a barrier before each timed launch, the MAX over ranks
of the median is reported by rank 0. Link bandwidth of the roofline: 900 GB/s per direction per GPU (NVLink 5 nominal);
a plain peer copy measured 770 GB/s on these boxes, which is given beside each row for context.
"""

from __future__ import annotations

import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS = 900.0          # roofline denominator
MEASURED_COPY_GBS = 770.0  # a plain peer-to-peer copy on these boxes (context)


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p.get("bf16_tflops_sustained", p["bf16_tflops"])
    return 6650.0, 1590.0


def timed(fn, iters=7, warmup=3):
    for _ in range(warmup):
        fn()
    out = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    t = torch.tensor([statistics.median(out)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from halo_b200.ops import _lib

    hbm, tf = peaks()
    rows = []
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    only = next((a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--only=")), "")
    out_path = args[0] if args else None

    def report(name, ms, flops=0.0, link_bytes=0.0, note=""):
        roof_ms = max(flops / (tf * 1e9) if flops else 0.0, link_bytes / (LINK_GBS * 1e6) if link_bytes else 0.0)
        rec = {"case": name, "ms": round(ms, 3), "roofline_ms": round(roof_ms, 3),
               "fraction_of_roofline": round(roof_ms / ms, 3) if ms else 0.0,
               "link_ms_at_measured_copy": round(link_bytes / (MEASURED_COPY_GBS * 1e6), 3) if link_bytes else 0.0, "note": note}
        rows.append(rec)
        if rank == 0:
            print(f"{name:44s} {ms:8.3f} ms   roofline {roof_ms:7.3f} ms   {rec['fraction_of_roofline']:5.2f}  {note}", flush=True)

    T, H = 65536, 2048
    if only in ("", "link"):
        bench_link(world, dev, report, timed)
    if only in ("", "tp"):
        bench_tensor_parallel(world, dev, report, timed, T, H)
    if only in ("", "zero"):
        bench_sharded_optimizer(world, dev, report, timed)
    if only in ("", "moe"):
        bench_moe_layer(world, dev, report, timed, T, H)
    _lib.raise_on_status(dev)
    if rank == 0 and out_path:
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        json.dump({"world": world, "link_gbs": LINK_GBS, "measured_copy_gbs": MEASURED_COPY_GBS, "bf16_tflops": tf, "rows": rows},
                  open(out_path, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


def bench_link(world, dev, report, timed):
    """What one GPU reaches towards ONE peer over NVLink with each access form, 1 GiB each way at once on every rank
    (rank r -> rank r+1): the copy engine, stores from a kernel, loads from a kernel. These are the practical ceilings
    of the fused kernels' transfers; the roofline column keeps the nominal 900 GB/s."""
    import torch.distributed._symmetric_memory as symm

    from halo_b200.ops import _lib

    n = 1 << 30
    buf = symm.empty((n,), dtype=torch.uint8, device=dev)
    hdl = symm.rendezvous(buf, dist.group.WORLD)
    src = torch.empty(n, dtype=torch.uint8, device=dev)
    rank = dist.get_rank()
    peer = (rank + 1) % world
    remote = hdl.get_buffer(peer, (n,), torch.uint8)
    L = _lib.lib()
    one = (_lib.c_void_p * 1)(int(hdl.buffer_ptrs[peer]))

    def ce_copy():
        remote.copy_(src)

    def kernel_stores():
        _lib.check(L.halo_broadcast_bytes(_lib.ptr(src), one, _lib.c_int(1), _lib.c_ll(0), _lib.c_ll(n), _lib.stream_ptr(dev)),
                   "halo_broadcast_bytes")

    def kernel_loads():
        _lib.check(L.halo_peer_pull(_lib.ptr(src), _lib.c_void_p(int(hdl.buffer_ptrs[peer])), _lib.c_ll(n), _lib.c_int(0),
                                    _lib.stream_ptr(dev)), "halo_peer_pull")

    for name, fn in (("1 GiB to one peer: copy engine", ce_copy), ("1 GiB to one peer: stores from a kernel", kernel_stores),
                     ("1 GiB from one peer: loads from a kernel", kernel_loads)):
        ms = timed(fn, iters=5, warmup=2)
        report(name, ms, 0.0, float(n), f"{n / ms / 1e6:.0f} GB/s per direction")
    hdl.barrier(channel=0)


def bench_tensor_parallel(world, dev, report, timed, T, H):
    from halo_b200.ops import gemm
    from halo_b200.parallel.tensor_parallel import TensorParallel, _all_gather_rows, row_parallel_linear

    # ---- row-parallel GEMM with the reduce-scatter's transfer in its epilogue (O-projection shape, TP = world) ----
    K = 4096 // world
    tp = TensorParallel(dist.group.WORLD, dev, hidden=H, max_tokens=T)
    x = (torch.randn(T, K, device=dev) * 0.05).bfloat16()
    w = (torch.randn(H, K, device=dev) * 0.05).bfloat16()
    flops = 2.0 * T * H * K
    link = (world - 1) / world * T * H * 2.0          # partial tiles this rank sends to the other owners
    ms = timed(lambda: row_parallel_linear(x, w, tp))
    report("fused GEMM + reduce-scatter (own kernels)", ms, flops, link, f"[{T}x{K}] x [{H}x{K}]^T, tp={world}")
    y_full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    y_shard = torch.empty(T // world, H, device=dev, dtype=torch.bfloat16)

    def baseline_rs():
        gemm.matmul(x, w, out=y_full)
        dist.reduce_scatter_tensor(y_shard, y_full)

    report("  baseline: own GEMM, then NCCL reduce-scatter", timed(baseline_rs), flops, link)

    # ---- sequence gather by peer pulls vs NCCL all-gather --------------------------------------------------------
    shard = (torch.randn(T // world, H, device=dev) * 0.05).bfloat16()
    link = (world - 1) / world * T * H * 2.0
    report("sequence gather by peer pulls", timed(lambda: _all_gather_rows(shard, tp)), 0.0, link)
    full = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    report("  baseline: NCCL all-gather", timed(lambda: dist.all_gather_into_tensor(full, shard)), 0.0, link)



def bench_sharded_optimizer(world, dev, report, timed):
    from halo_b200.parallel.zero import FusedShardedAdamW

    # ---- reduce-scatter + AdamW + all-gather of the replicated parameters (1.4 B parameters) -----------------------
    n = 1_400_000_000 // 8 * 8
    p = torch.nn.Parameter(torch.zeros(n, device=dev, dtype=torch.bfloat16))
    opt = FusedShardedAdamW([("flat", p)], dist.group.WORLD, dev, lr=1e-4)
    p.grad = torch.full((n,), 1e-3, device=dev, dtype=torch.bfloat16)
    one = torch.ones(1, device=dev)
    zero = torch.zeros(1, device=dev, dtype=torch.int32)

    def fused_step():
        opt.pack_and_reduce()
        opt.step(one, zero)

    link = 2.0 * (world - 1) / world * n * 2.0        # gradient slice in from every peer, weight slice out to every peer
    ms = timed(fused_step, iters=5, warmup=2)
    report("reduce-scatter + AdamWBF16 + all-gather (two kernels)", ms, 0.0, link, f"{n / 1e9:.1f} B bf16 parameters")
    g = p.grad

    def baseline_zero():
        dist.all_reduce(g)

    report("  baseline: NCCL all-reduce of the gradients alone", timed(baseline_zero, iters=5, warmup=2), 0.0, link)
    del opt, p, g



def bench_moe_layer(world, dev, report, timed, T, H):
    """One MoE layer at the 30B-A3B shapes (128 experts of FFN 768, top-8, EP = world), forward and forward + backward,
    with the token movement inside the GEMM kernels and as separate push / pull kernels."""
    from halo_b200.ops.moe import moe_experts, router_topk
    from halo_b200.parallel.runtime import SymmetricTransport

    E, F, topk = 128, 768, 8
    xm = (torch.randn(T, H, device=dev) * 0.05).bfloat16()
    idx, wts = router_topk(torch.randn(T, E, device=dev), topk, True)
    wgu = (torch.randn(E // world, 2 * F, H, device=dev) * 0.05).bfloat16()
    wdn = (torch.randn(E // world, H, F, device=dev) * 0.05).bfloat16()
    gout = (torch.randn(T, H, device=dev) * 0.05).bfloat16()
    fwd_flops = 2.0 * T * topk * 3 * H * F
    one_way = (world - 1) / world * T * topk * H * 2.0          # rows out to the experts, or back
    for fused in (True, False):
        tr = SymmetricTransport(dist.group.WORLD, dev)
        tr.fused = fused
        tr.configure(max_tokens=T, top_k=topk, hidden=H, n_local_experts=E // world)
        name = "movement inside the GEMM kernels" if fused else "separate push / pull kernels"
        with torch.no_grad():
            ms = timed(lambda: moe_experts(xm, idx, wts, wgu, wdn, tr), iters=5, warmup=2)
        # with the movement inside the kernels both directions overlap the products: the bound is the slower of the GEMMs
        # and the two transfers
        report(f"MoE layer forward, {name}", ms, fwd_flops, 2.0 * one_way, "roofline: the slower of the GEMMs and the two transfers")

        def fwd_bwd():
            xa = xm.detach().requires_grad_()
            wa, wb = wgu.detach().requires_grad_(), wdn.detach().requires_grad_()
            moe_experts(xa, idx, wts, wa, wb, tr).backward(gout)

        ms = timed(fwd_bwd, iters=5, warmup=2)
        report(f"MoE layer forward + backward, {name}", ms, 3.0 * fwd_flops, 4.0 * one_way)
        if fused:
            # one more pass with a CUDA event after every phase: where the time goes (this rank's stream)
            from halo_b200.ops import moe as moe_ops

            moe_ops.PHASE_MARKS = []
            dist.barrier()
            fwd_bwd()
            torch.cuda.synchronize()
            marks, moe_ops.PHASE_MARKS = moe_ops.PHASE_MARKS, None
            if dist.get_rank() == 0:
                for (_, a), (label, b) in zip(marks, marks[1:]):
                    if label != "start":
                        print(f"    {label:44s} {a.elapsed_time(b):7.3f} ms", flush=True)
        del tr
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
