"""Kernel microbenchmarks at the shapes of the 30B-A3B MoE layer (64k-token packed rows).

    python benchmarks/kernels.py                    # every case, full shapes
    python benchmarks/kernels.py --only gemm attn   # a subset
    python benchmarks/kernels.py --small --iters 1 --warmup 1 --only gemm_qkv   # a case sized for a profiler capture

Timing: CUDA events on the launching stream around each call, after warm-up, with a write of a buffer
larger than L2 between iterations; the median is reported. Rates are set against the measured copy
bandwidth and bf16 GEMM rate of the machine when a ``MEASURED_PEAKS.json`` is found at the repository
root (else against 6.65 TB/s and 1.59 PFLOP/s).

Covers what the reference's kernel benchmarks cover (tests/gpu/profiling/benchmark_roofline.py,
benchmark_grouped_mm.py, benchmark_moe_block.py, benchmark_attention_implementations.py).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from halo_b200.data.packing import sample_doc_lengths  # noqa: E402
from halo_b200.ops import attention as attn_ops  # noqa: E402
from halo_b200.ops import gemm, moe as moe_ops  # noqa: E402
from halo_b200.ops.norm import add_rms_norm, rms_norm  # noqa: E402

import numpy as np  # noqa: E402


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


class Timer:
    def __init__(self, iters, warmup):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn):
        for _ in range(self.warmup):
            fn()
        times = []
        for _ in range(self.iters):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        return statistics.median(times)


def bf16(*shape):
    return torch.randn(*shape, device="cuda", dtype=torch.bfloat16) * 0.05


def cases(small: bool):
    T = 8192 if small else 65536
    H, F, E, K = 2048, 768, 128, 8
    NQ, NKV, HD = 32, 4, 128
    V = 16384 if small else 151936
    out = {}

    # ---- dense GEMMs --------------------------------------------------------------------------
    def dense(name, M, N, Kd, a_t=False, b_t=True):
        a = bf16(Kd, M) if a_t else bf16(M, Kd)
        b = bf16(N, Kd) if b_t else bf16(Kd, N)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        out[name] = (lambda: gemm.matmul(a, b, a_t=a_t, b_t=b_t, out=c), 2.0 * M * N * Kd, 2.0 * (M * Kd + N * Kd + M * N))

    dense("gemm_qkv", T, (NQ + 2 * NKV) * HD, H)
    dense("gemm_o", T, H, NQ * HD)
    dense("gemm_qkv_dgrad", T, H, (NQ + 2 * NKV) * HD, b_t=False)
    dense("gemm_qkv_wgrad", (NQ + 2 * NKV) * HD, H, T, a_t=True, b_t=False)
    dense("gemm_head", T, V, H)
    dense("gemm_square_8192", 8192, 8192, 8192)

    def cublas(name, M, N, Kd):
        a, b = bf16(M, Kd), bf16(N, Kd)
        out[name] = (lambda: torch.matmul(a, b.t()), 2.0 * M * N * Kd, 2.0 * (M * Kd + N * Kd + M * N))

    cublas("cublas_qkv", T, (NQ + 2 * NKV) * HD, H)
    cublas("cublas_square_8192", 8192, 8192, 8192)

    # ---- routed experts (single rank holds all experts) ----------------------------------------
    x = bf16(T, H)
    logits = torch.randn(T, E, device="cuda", dtype=torch.bfloat16)
    idx, w = moe_ops.router_topk(logits, K, True)
    w_gu, w_dn = bf16(E, 2 * F, H), bf16(E, H, F)
    expert_flops = 2.0 * T * K * 3 * H * F
    out["moe_experts_fwd"] = (lambda: moe_ops.moe_experts(x, idx, w, w_gu, w_dn), expert_flops,
                              2.0 * (2 * T * H + 2 * T * K * (2 * H + F) + 3 * E * H * F))

    xg = x.clone().requires_grad_(True)
    wg, wd = w_gu.clone().requires_grad_(True), w_dn.clone().requires_grad_(True)
    dy = bf16(T, H)

    def moe_fb():
        y = moe_ops.moe_experts(xg, idx, w, wg, wd)
        y.backward(dy)
        xg.grad = wg.grad = wd.grad = None

    out["moe_experts_fwd_bwd"] = (moe_fb, 3 * expert_flops, 0.0)

    # experts with bias vectors around a clamped GLU (the gpt-oss form): the same grouped products with the bias /
    # activation row kernels between them (separate-kernel pipeline)
    from halo_b200.ops.biased_glu_experts import GLU_ALPHA

    b_gu, b_dn = bf16(E, 2 * F).requires_grad_(True), bf16(E, H).requires_grad_(True)
    out["moe_glu_experts_fwd"] = (lambda: moe_ops.moe_experts(x, idx, w, w_gu, w_dn, glu=(b_gu.detach(), b_dn.detach(), 7.0, GLU_ALPHA)),
                                  expert_flops, 0.0)

    def moe_glu_fb():
        y = moe_ops.moe_experts(xg, idx, w, wg, wd, glu=(b_gu, b_dn, 7.0, GLU_ALPHA))
        y.backward(dy)
        xg.grad = wg.grad = wd.grad = b_gu.grad = b_dn.grad = None

    out["moe_glu_experts_fwd_bwd"] = (moe_glu_fb, 3 * expert_flops, 0.0)

    # ---- attention ----------------------------------------------------------------------------
    for dist_name in ("chat", "loguniform"):
        lens = sample_doc_lengths(T, np.random.default_rng(0), dist_name)
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        plan = attn_ops.build_plan(cu, "cuda")
        q, k, v = bf16(T, NQ * HD), bf16(T, NKV * HD), bf16(T, NKV * HD)
        flops = sum(4.0 * NQ * HD * (n * (n + 1) / 2) for n in lens)
        out[f"attn_fwd_{dist_name}"] = (lambda q=q, k=k, v=v, plan=plan: attn_ops.flash_attention(q, k, v, plan, NQ, NKV),
                                       flops, 2.0 * T * HD * (2 * NQ + 2 * NKV))
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        do = bf16(T, NQ * HD)

        def attn_fb(qg=qg, kg=kg, vg=vg, plan=plan, do=do):
            o = attn_ops.flash_attention(qg, kg, vg, plan, NQ, NKV)
            o.backward(do)
            qg.grad = kg.grad = vg.grad = None

        out[f"attn_fwd_bwd_{dist_name}"] = (attn_fb, 3.5 * flops, 0.0)

    # sliding window of 4096 tokens over one document as long as the batch: the work lists drop key tiles left of the
    # window, so the count of useful flops is the band's, not the triangle's
    win = 4096 if not small else 1024
    cu_w = np.array([0, T], dtype=np.int64)
    plan_w = attn_ops.build_plan(cu_w, "cuda", window=win)
    band = sum(min(i + 1, win) for i in range(T))
    flops_w = 4.0 * NQ * HD * band
    qw, kw, vw = (bf16(T, n * HD).requires_grad_(True) for n in (NQ, NKV, NKV))
    do_w = bf16(T, NQ * HD)
    out["attn_fwd_window"] = (lambda: attn_ops.flash_attention(qw.detach(), kw.detach(), vw.detach(), plan_w, NQ, NKV),
                              flops_w, 2.0 * T * HD * (2 * NQ + 2 * NKV))

    def attn_w_fb():
        o = attn_ops.flash_attention(qw, kw, vw, plan_w, NQ, NKV)
        o.backward(do_w)
        qw.grad = kw.grad = vw.grad = None

    out["attn_fwd_bwd_window"] = (attn_w_fb, 3.5 * flops_w, 0.0)

    # ---- bandwidth-bound pieces ---------------------------------------------------------------
    wn = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    res = bf16(T, H)
    out["rmsnorm_fwd"] = (lambda: rms_norm(x, wn, 1e-6), 0.0, 2.0 * 2 * T * H)
    out["add_rmsnorm_fwd"] = (lambda: add_rms_norm(x, res, wn, 1e-6), 0.0, 2.0 * 4 * T * H)
    big = torch.empty(1 << 30, dtype=torch.bfloat16, device="cuda") if not small else torch.empty(1 << 27, dtype=torch.bfloat16, device="cuda")
    big2 = torch.empty_like(big)
    out["copy_reference"] = (lambda: big2.copy_(big), 0.0, 2.0 * 2 * big.numel())

    # ---- optimizer steps on one large tensor: bf16 moments (14 bytes moved per parameter) and 8-bit moments with 24-bit
    # weights (12 bytes per parameter) ------------------------------------------------------------
    from halo_b200.optim.adamw_bf16 import AdamWBF16
    from halo_b200.optim.adamw_q8 import AdamWQ8

    n_opt = (1 << 25) if small else (1 << 28)
    for label, cls, moved in (("adamw_bf16_step", AdamWBF16, 14.0), ("adamw_q8_step", AdamWQ8, 12.0)):
        p_opt = torch.nn.Parameter(bf16(n_opt))
        p_opt.grad = bf16(n_opt)
        opt = cls([("w", p_opt)], lr=1e-4)
        opt.step()                                   # state allocation outside the timed calls
        out[label] = (opt.step, 0.0, moved * n_opt)
    return out


def family_cases(small: bool):
    """Bandwidth-bound kernels of the other families and of generation (run with ``--families``): residual-stream ops
    at 4 streams, per-stream norm, block-scaled fake quantisation, standalone SwiGLU, decode attention over a cache, 4-bit dequantisation of an expert bank."""
    from halo_b200.inference.generate import KVCache
    from halo_b200.ops import lowp, streams
    from halo_b200.ops.activation import swiglu

    T = 8192 if small else 32768
    H, N = 2048, 4
    out = {}
    st, blk = bf16(T, N, H), bf16(T, H)
    w = torch.rand(T, N, device="cuda")
    comb = torch.softmax(torch.randn(T, N, N, device="cuda"), dim=-1)
    with torch.no_grad():
        out["stream_collapse_fwd"] = (lambda: streams.collapse_streams(st, w), 0.0, 2.0 * T * H * (N + 1))
        out["stream_mix_fwd"] = (lambda: streams.mix_streams(blk, st, w, comb), 0.0, 2.0 * T * H * (2 * N + 1))
        out["stream_inject_fwd"] = (lambda: streams.inject_streams(blk, st, w), 0.0, 2.0 * T * H * (2 * N + 1))
        out["sinkhorn_20_iters"] = (lambda: streams.sinkhorn_knopp(comb, 20, 1e-6), 0.0, 4.0 * 2 * T * N * N)
        wide, nw = bf16(T, N * H), torch.zeros(N * H, device="cuda")
        out["grouped_rmsnorm_fwd"] = (lambda: streams.grouped_rms_norm(wide, nw, 1e-6, N), 0.0, 2.0 * 2 * T * N * H)
        for fmt in lowp.FORMATS:
            out[f"fake_quant_{fmt}"] = (lambda fmt=fmt: lowp.fake_quant(wide, fmt), 0.0, 2.0 * 2 * T * N * H)
        pre = bf16(T, 2 * 6144)
        out["swiglu_fwd"] = (lambda: swiglu(pre), 0.0, 2.0 * 3 * T * 6144)
        B, S, NQ, NKV, HD = (16, 2048, 32, 4, 128) if small else (64, 8192, 32, 4, 128)
        cache = KVCache(1, B, S, NKV, HD, torch.bfloat16, "cuda")
        cache.k.normal_()
        cache.v.normal_()
        cache.lengths.fill_(S - 1)
        cache.begin_decode()
        q = bf16(B, NQ * HD)
        out["decode_attention"] = (lambda: cache.attend(0, q, NQ), 4.0 * B * NQ * HD * S, 2.0 * 2 * B * S * NKV * HD)
        from halo_b200.ops import nf4

        E, F = (32, 768) if small else (128, 768)              # one layer's gate/up expert bank of the 30B-A3B shape
        packed = nf4.quantize_4bit(bf16(E, 2 * F, H), "nf4", nested=False)
        out["dequant_nf4_expert_bank"] = (lambda: nf4.dequantize_4bit(packed), 0.0, (0.5 + 4.0 / 64 + 2.0) * E * 2 * F * H)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--families", action="store_true", help="the other families' kernels and decode attention instead of the flagship's")
    ap.add_argument("--only", nargs="*", default=None, help="substrings of case names to run")
    ap.add_argument("--small", action="store_true", help="8k tokens, 16k vocabulary: sized for a profiler capture")
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    hbm, tf, tag = peaks()
    timer = Timer(args.iters, args.warmup)
    rows = []
    for name, (fn, flops, nbytes) in (family_cases(args.small) if args.families else cases(args.small)).items():
        if args.only and not any(s in name for s in args.only):
            continue
        ms = timer(fn)
        tfs = flops / ms / 1e9 if flops else 0.0
        gbs = nbytes / ms / 1e6 if nbytes else 0.0
        frac = max(tfs / tf, gbs / hbm)
        rows.append({"case": name, "ms": round(ms, 4), "tflops": round(tfs, 1), "gb_s": round(gbs, 1),
                     "fraction_of_peak": round(frac, 3)})
        print(f"{name:28s} {ms:9.3f} ms  {tfs:8.1f} TF/s  {gbs:8.1f} GB/s  {frac:5.2f} {tag}", flush=True)
    if args.json:
        os.makedirs(os.path.dirname(args.json) or ".", exist_ok=True)
        json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "basis": tag}, "rows": rows}, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
