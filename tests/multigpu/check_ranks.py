"""Run under torchrun on 2+ GPUs: the expert transport over peer memory, the fused sharded optimizer,
the peer-store broadcast and context-parallel attention against single-device references. Prints ``CHECKS PASSED`` on rank 0."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def close(a, b, tol, what):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * ref + 1e-3, f"{what}: max err {err} (ref max {ref})"


def check_expert_transport(tr, dev, rank, world, what):
    """Each rank owns E/world experts; every rank's tokens must come back as if all experts were local. Three calls in
    a row through one transport, with a different number of tokens on every rank and call."""
    for call in range(3):
        _check_expert_call(tr, dev, rank, world, f"{what}, call {call}", 1536 - 128 * ((rank + call) % 3), call)


def _check_expert_call(tr, dev, rank, world, what, T, call):
    from halo_b200.ops.moe import moe_experts, moe_ffn_reference

    H, F, E, k = 512, 256, 16, 4
    g = torch.Generator(device=dev).manual_seed(7)
    wgu_full = (torch.randn(E, 2 * F, H, device=dev, generator=g) * 0.05).bfloat16()
    wd_full = (torch.randn(E, H, F, device=dev, generator=g) * 0.05).bfloat16()
    g2 = torch.Generator(device=dev).manual_seed(100 + rank + 17 * call)
    x = torch.randn(T, H, device=dev, generator=g2).bfloat16()
    scores = torch.rand(T, E, device=dev, generator=g2)
    w, idx = torch.topk(scores, k, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).float()
    idx = idx.to(torch.int32)
    e0, e1 = rank * (E // world), (rank + 1) * (E // world)
    xa, wa = x.clone().requires_grad_(), w.clone().requires_grad_()
    wgu = wgu_full[e0:e1].clone().requires_grad_()
    wd = wd_full[e0:e1].clone().requires_grad_()
    out = moe_experts(xa, idx, wa, wgu, wd, tr)
    gout = torch.randn(T, H, device=dev, generator=g2).bfloat16()
    out.backward(gout)
    torch.cuda.synchronize()
    # reference: all experts local, this rank's tokens
    xb, wb = x.float().requires_grad_(), w.clone().requires_grad_()
    wgub, wdb = wgu_full.float().requires_grad_(), wd_full.float().requires_grad_()
    ref = moe_ffn_reference(xb, idx, wb, wgub, wdb)
    ref.backward(gout.float())
    close(out, ref, 3e-2, f"ep out ({what})")
    close(xa.grad, xb.grad, 4e-2, f"ep dx ({what})")
    close(wa.grad, wb.grad, 4e-2, f"ep dw_route ({what})")
    # expert weight gradients: sum over ranks of the reference's per-rank contributions
    gw = wgub.grad.clone()
    gd = wdb.grad.clone()
    dist.all_reduce(gw)
    dist.all_reduce(gd)
    close(wgu.grad, gw[e0:e1], 5e-2, f"ep dw_gate_up ({what})")
    close(wd.grad, gd[e0:e1], 5e-2, f"ep dw_down ({what})")


def check_biased_glu_experts(tr, dev, rank, world):
    """Experts with bias vectors around a clamped GLU, sharded over the ranks (whole experts with their bias rows): output
    and gradients of this rank's tokens against the dense fp32 form over ALL experts. Gradients are compared by norm: a
    pre-activation within a rounding step of the clamp can fall on either side in two correct summation orders."""
    from halo_b200.ops.biased_glu_experts import GLU_ALPHA, biased_glu_experts_reference
    from halo_b200.ops.moe import moe_experts

    H, F, E, k, T, limit = 512, 256, 16, 4, 1536 - 128 * (rank % 3), 2.0
    g = torch.Generator(device=dev).manual_seed(11)
    wgu_full = (torch.randn(E, 2 * F, H, device=dev, generator=g) * 0.08).bfloat16()
    wd_full = (torch.randn(E, H, F, device=dev, generator=g) * 0.05).bfloat16()
    bgu_full = (torch.randn(E, 2 * F, device=dev, generator=g) * 0.5).bfloat16()
    bd_full = (torch.randn(E, H, device=dev, generator=g) * 0.5).bfloat16()
    g2 = torch.Generator(device=dev).manual_seed(300 + rank)
    x = torch.randn(T, H, device=dev, generator=g2).bfloat16()
    w, idx = torch.topk(torch.rand(T, E, device=dev, generator=g2), k, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).float()
    idx = idx.to(torch.int32)
    e0, e1 = rank * (E // world), (rank + 1) * (E // world)
    mine = [t.detach().clone().requires_grad_() for t in (x, w, wgu_full[e0:e1], wd_full[e0:e1], bgu_full[e0:e1], bd_full[e0:e1])]
    out = moe_experts(mine[0], idx, mine[1], mine[2], mine[3], tr, glu=(mine[4], mine[5], limit, GLU_ALPHA))
    gout = torch.randn(T, H, device=dev, generator=g2).bfloat16()
    out.backward(gout)
    torch.cuda.synchronize()
    full = [t.detach().float().requires_grad_() for t in (x, w.clone(), wgu_full, wd_full, bgu_full, bd_full)]
    ref = biased_glu_experts_reference(full[0], idx, full[1], full[2], full[4], full[3], full[5], limit, stored_dtype=torch.bfloat16)
    ref.backward(gout.float())
    close(out, ref, 3e-2, "biased glu ep out")
    wants = [full[0].grad, full[1].grad]
    for t in full[2:]:
        gsum = t.grad.clone()
        dist.all_reduce(gsum)                       # a bank's gradient collects every rank's tokens
        wants.append(gsum[e0:e1])
    for got, want, name in zip(mine, wants, ("dx", "dw_route", "dw_gate_up", "dw_down", "db_gate_up", "db_down")):
        diff = got.grad.float() - want
        assert diff.norm().item() <= 2e-2 * want.norm().item() + 1e-6, f"biased glu ep {name}: {diff.norm().item()} of {want.norm().item()}"


def check_fused_optimizer(dev, rank, world):
    from halo_b200.optim.adamw_bf16 import adamw_bf16_step_reference, param_name_hash, SR_KEY
    from halo_b200.parallel.zero import FusedShardedAdamW

    shapes = {"a.weight": (300, 64), "b.norm": (64,), "c.weight": (1000, 33), "d.weight": (7,)}
    g = torch.Generator().manual_seed(3)
    init = {n: torch.randn(s, generator=g).bfloat16() for n, s in shapes.items()}
    params = [(n, torch.nn.Parameter(t.clone().to(dev))) for n, t in init.items()]
    opt = FusedShardedAdamW(params, dist.group.WORLD, dev, lr=1e-2, weight_decay=0.1)
    ref_p = {n: t.clone() for n, t in init.items()}
    ref_m = {n: torch.zeros_like(t) for n, t in init.items()}
    ref_v = {n: torch.zeros_like(t) for n, t in init.items()}
    for step in range(1, 4):
        grads_all = []
        for r in range(world):
            gr = torch.Generator().manual_seed(1000 * step + r)
            grads_all.append({n: (torch.randn(s, generator=gr) * 0.1).bfloat16() for n, s in shapes.items()})
        for n, p in params:
            p.grad = grads_all[rank][n].to(dev)
        sq = opt.pack_and_reduce()
        dist.all_reduce(sq)
        total = {n: sum(ga[n].float() for ga in grads_all) for n in shapes}
        want_sq = sum(t.pow(2).sum() for t in total.values())
        assert abs(sq.item() - want_sq.item()) <= 1e-3 * want_sq.item(), (sq.item(), want_sq.item())
        scale = torch.tensor([0.5], device=dev)
        opt.step(scale, None)
        torch.cuda.synchronize()
        b1, b2 = 0.9, 0.999
        for n in shapes:
            wd = 0.1 if len(shapes[n]) > 1 else 0.0
            adamw_bf16_step_reference(ref_p[n], total[n], ref_m[n], ref_v[n], beta1=b1, beta2=b2,
                                      step_size=1e-2 / (1 - b1**step), bc2_sqrt=(1 - b2**step) ** 0.5, eps=1e-8,
                                      wd_factor=1.0 - 1e-2 * wd, key=SR_KEY, step=step, name_hash=param_name_hash(n),
                                      grad_scale=0.5)
        for n, p in params:
            assert torch.equal(p.detach().cpu(), ref_p[n]), f"fused optimizer: {n} differs at step {step} on rank {rank}"


def check_broadcast_and_allreduce(dev, rank, world):
    import torch.distributed._symmetric_memory as symm

    from halo_b200.ops import _lib

    n = 1 << 20
    buf = symm.empty((n,), dtype=torch.bfloat16, device=dev)
    buf.zero_()
    h = symm.rendezvous(buf, dist.group.WORLD)
    h.barrier(channel=0)
    src = torch.arange(n, device=dev, dtype=torch.float32).bfloat16()
    L = _lib.lib()
    if rank == 0:
        ptrs = (_lib.c_void_p * world)(*list(h.buffer_ptrs))
        _lib.check(L.halo_broadcast_bytes(_lib.ptr(src), ptrs, _lib.c_int(world), _lib.c_ll(0), _lib.c_ll(n * 2),
                                          _lib.stream_ptr(dev)), "halo_broadcast_bytes")
    h.barrier(channel=0)
    torch.cuda.synchronize()
    assert torch.equal(buf, src), "broadcast payload differs"
    small = symm.empty((64,), dtype=torch.float32, device=dev)
    small.fill_(float(rank + 1))
    hs = symm.rendezvous(small, dist.group.WORLD)
    hs.barrier(channel=0)
    out = torch.empty(64, device=dev)
    ptrs = (_lib.c_void_p * world)(*list(hs.buffer_ptrs))
    _lib.check(L.halo_allreduce_small(ptrs, _lib.c_int(world), _lib.ptr(out), _lib.c_int(64), _lib.stream_ptr(dev)),
               "halo_allreduce_small")
    torch.cuda.synchronize()
    assert torch.all(out == world * (world + 1) / 2)
    hs.barrier(channel=0)


def check_sharded_weight_push(dev, rank, world):
    """First half of the ranks train (expert banks cut over them), second half receive a full copy: every trainer stores
    its slice and its share of the replicated tensors straight into the receivers' arenas."""
    from halo_b200.weight_sync.group import ShardedCopySync

    n_train = world // 2
    trainers, rollouts = list(range(n_train)), list(range(n_train, world))
    E = 4 * n_train
    manifest = [("embed", (64, 48), torch.bfloat16), ("norm", (48,), torch.float32), ("bank_a", (E, 24, 48), torch.bfloat16),
                ("head", (64, 48), torch.bfloat16), ("bank_b", (E, 48, 8), torch.bfloat16)]
    full = {}
    g = torch.Generator().manual_seed(99)                      # the same full tensors on every rank
    for name, shape, dtype in manifest:
        full[name] = torch.randn(shape, generator=g).to(dtype).to(dev)
    sync = ShardedCopySync(dist.group.WORLD, dev, manifest, trainers, rollouts)
    sync.arena.zero_()
    pieces = []
    if rank in trainers:
        t = trainers.index(rank)
        e = E // n_train
        for k, name in enumerate(("embed", "norm", "head")):
            if sync.owner_of_replicated(k) == t:
                pieces.append((name, full[name], 0))
        for name in ("bank_a", "bank_b"):
            pieces.append((name, full[name][t * e:(t + 1) * e], t * e))
    for _ in range(2):
        sync.push(pieces)
    if rank in rollouts:
        for name, shape, dtype in manifest:
            assert torch.equal(sync.view(name, shape, dtype), full[name]), f"sharded weight push: {name} differs"


def check_zero3_layers(dev, rank, world):
    """Decoder-layer matrices as 1 / N slices: the pull-gather rebuilds every layer's matrices bit for bit, the per-layer
    reduce-scatter gives every rank the fp32 sum of its slice, and two training steps follow the replicated model."""
    import dataclasses

    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.optim.factory import build_optimizer
    from halo_b200.parallel.runtime import ParallelRuntime
    from halo_b200.parallel.zero3 import shard_layers
    from halo_b200.trainers.engine import TrainEngine

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=3, num_experts=0, intermediate_size=256)

    def run(sharded):
        model = build_model(cfg, device=dev, dtype=torch.bfloat16, seed=21, gradient_checkpointing=True)
        originals = {n: p.detach().clone() for n, p in model.named_parameters()}
        zero3 = shard_layers(model, dist.group.WORLD, dev) if sharded else None
        if sharded:
            for li in range(len(model.layers)):
                zero3.before_layer(li, backward=False)
                for name, p, *_ in zero3.params[li]:
                    assert torch.equal(p.detach(), originals[name]), f"gathered {name} differs"
                zero3.after_layer(li, backward=False)
            # a reduce-scatter of known values: every rank writes (rank + 1) everywhere, each slice sums to N (N + 1) / 2
            zero3.before_layer(1, backward=True)
            for _, p, *_ in zero3.params[1]:
                p.grad.fill_(float(rank + 1))
            zero3.after_layer(1, backward=True)
            torch.cuda.synchronize()
            n = zero3.layer_len[1] // world
            got = zero3.grad_shard[zero3.shard_off[1]:zero3.shard_off[1] + n]
            lo = rank * n
            used = sum(((num + 7) // 8 * 8) for _, _, _, num, _ in zero3.params[1])
            want = torch.zeros_like(got)
            # padding between tensors and at the layer's end stays zero
            for _, _, at, num, _ in zero3.params[1]:
                a, b = max(at, lo), min(at + num, lo + n)
                if a < b:
                    want[a - lo:b - lo] = world * (world + 1) / 2
            assert torch.equal(got, want), "reduce-scatter of a layer's gradients differs"
            assert used <= zero3.layer_len[1]
            zero3.after_step()
        opt = build_optimizer(model, "adamw_bf16", lr=1e-3, weight_decay=0.01)
        eng = TrainEngine(model, opt, dev, max_grad_norm=1.0, parallel=ParallelRuntime(dev, dp_group=dist.group.WORLD))
        out = []
        for step in range(3):
            b = synthetic_packed_batch(2048, cfg.vocab_size, seed=50 * rank + step)
            o = eng.train_step(b)
            t = o.loss.detach().float().clone()
            dist.all_reduce(t)
            out.append((float(t), float(o.grad_norm)))
        return out

    want, got = run(False), run(True)
    assert abs(want[0][0] - got[0][0]) < 2e-3 and abs(want[0][1] - got[0][1]) < 2e-2 * want[0][1], (want, got)
    for (lw, nw), (lg, ng) in zip(want, got):
        assert abs(lw - lg) < 3e-2, (want, got)       # bf16 weights, differently keyed rounding noise after the first update


def check_nvls_forms(dev, rank, world):
    """The multimem forms (in-switch reduction, multicast stores) against the plain peer forms, where the symmetric
    buffers are bound to an NVLink multicast object; skipped (and said so) where they are not."""
    import torch.distributed._symmetric_memory as symm

    from halo_b200.ops import _lib
    from halo_b200.optim.adamw_bf16 import adamw_bf16_step_reference, param_name_hash, SR_KEY
    from halo_b200.parallel.zero import FusedShardedAdamW

    n = 1 << 18
    buf = symm.empty((n,), dtype=torch.float32, device=dev)
    h = symm.rendezvous(buf, dist.group.WORLD)
    mc = int(getattr(h, "multicast_ptr", 0) or 0)
    if not mc:
        if rank == 0:
            print("NVLS forms skipped: the symmetric buffers have no multicast binding on this box")
        return False
    L = _lib.lib()
    buf.copy_(torch.arange(n, device=dev, dtype=torch.float32) % 97 + rank)
    h.barrier(channel=0)
    out = torch.empty(4096, device=dev)
    _lib.check(L.halo_allreduce_small_mc(_lib.c_void_p(mc), _lib.ptr(out), _lib.c_int(4096), _lib.stream_ptr(dev)), "allreduce mc")
    torch.cuda.synchronize()
    want = (torch.arange(4096, device=dev, dtype=torch.float32) % 97) * world + world * (world - 1) / 2
    assert torch.equal(out, want), "multimem all-reduce"
    h.barrier(channel=0)
    src = (torch.arange(n, device=dev, dtype=torch.float32) * 3 + 1)
    if rank == 0:
        _lib.check(L.halo_broadcast_bytes_mc(_lib.ptr(src), _lib.c_void_p(mc), _lib.c_ll(0), _lib.c_ll(n * 4), _lib.stream_ptr(dev)),
                   "broadcast mc")
    torch.cuda.synchronize()
    h.barrier(channel=0)
    torch.cuda.synchronize()
    assert torch.equal(buf, src), "multimem broadcast"
    h.barrier(channel=0)
    # the sharded optimizer through the switch: gradient sums arrive rounded to bf16, everything else as usual
    shapes = {"a.weight": (300, 64), "b.norm": (64,), "c.weight": (1000, 33)}
    g = torch.Generator().manual_seed(3)
    init = {k: torch.randn(s, generator=g).bfloat16() for k, s in shapes.items()}
    params = [(k, torch.nn.Parameter(t.clone().to(dev))) for k, t in init.items()]
    opt = FusedShardedAdamW(params, dist.group.WORLD, dev, lr=1e-2, weight_decay=0.1, nvls=True)
    assert opt.nvls
    ref_p = {k: t.clone() for k, t in init.items()}
    ref_m = {k: torch.zeros_like(t) for k, t in init.items()}
    ref_v = {k: torch.zeros_like(t) for k, t in init.items()}
    for step in range(1, 3):
        grads_all = []
        for r in range(world):
            gr = torch.Generator().manual_seed(1000 * step + r)
            grads_all.append({k: (torch.randn(s, generator=gr) * 0.1).bfloat16() for k, s in shapes.items()})
        for k, p in params:
            p.grad = grads_all[rank][k].to(dev)
        opt.pack_and_reduce()
        opt.step(torch.tensor([0.5], device=dev), None)
        torch.cuda.synchronize()
        b1, b2 = 0.9, 0.999
        for k in shapes:
            total = sum(ga[k].float() for ga in grads_all).bfloat16().float()      # what the switch hands back
            adamw_bf16_step_reference(ref_p[k], total, ref_m[k], ref_v[k], beta1=b1, beta2=b2, step_size=1e-2 / (1 - b1**step),
                                      bc2_sqrt=(1 - b2**step) ** 0.5, eps=1e-8, wd_factor=1.0 - 1e-2 * (0.1 if len(shapes[k]) > 1 else 0.0),
                                      key=SR_KEY, step=step, name_hash=param_name_hash(k), grad_scale=0.5)
        for k, p in params:
            # the switch may add the ranks' values in another order than the reference: compare within a bf16 ulp or two
            close(p.detach().cpu(), ref_p[k], 2e-2, f"sharded optimizer through the switch: {k}, step {step}")
    return True


def check_context_parallel(dev, rank, world):
    """Attention of this rank's pieces of a packed row (keys and values read from their owners inside the kernels, foreign
    dK / dV returned through the staging buffers) against the flash kernel run on the whole row by one GPU, forward and
    backward; with paired early / late pieces and with contiguous chunks, on chat-length documents and on one long one."""
    import numpy as np

    from halo_b200.ops import attention as attn_ops
    from halo_b200.parallel.context_parallel import CPExchange, TILE, build_cp_plan, cp_attention, make_layout

    Hq, Hkv, D = 8, 2, 128
    total = 2048 * world
    rng = np.random.default_rng(5)
    lens, left = [], total
    while left > 0:
        n = int(min(left, rng.integers(100, 3000)))
        lens.append(n)
        left -= n
    exchanges = {False: CPExchange(dist.group.WORLD, dev, total // world + 4 * TILE, total + TILE, 2 * Hkv * D, direct_reads=False),
                 True: CPExchange(dist.group.WORLD, dev, total // world + 4 * TILE, total + TILE, 2 * Hkv * D, direct_reads=True)}
    chat = np.concatenate([[0], np.cumsum(lens)])
    for cu, balance, direct in ((chat, True, False), (np.array([0, total]), True, False), (chat, False, False),
                                (chat, True, True), (np.array([0, total]), True, True)):
        ex = exchanges[direct]
        g = torch.Generator(device=dev).manual_seed(11)              # same data on every rank
        q = (torch.randn(total, Hq * D, device=dev, generator=g) * 0.5).bfloat16()
        k = (torch.randn(total, Hkv * D, device=dev, generator=g) * 0.5).bfloat16()
        v = (torch.randn(total, Hkv * D, device=dev, generator=g) * 0.5).bfloat16()
        do = (torch.randn(total, Hq * D, device=dev, generator=g) * 0.5).bfloat16()
        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
        ref = attn_ops.flash_attention(qf, kf, vf, attn_ops.build_plan(cu, dev), Hq, Hkv)
        ref.backward(do)
        lay = make_layout(cu, rank, world, balance)
        idx = torch.from_numpy(lay.local_index()).to(dev)
        ql, kl, vl = (t[idx].clone().requires_grad_() for t in (q, k, v))
        plan = build_cp_plan(lay, dev)
        out = cp_attention(ql, kl, vl, lay, plan, dist.group.WORLD, ex, Hq, Hkv)
        if not direct and len(cu) == 2:
            # another exchange in between (as without recomputation): the backward must fetch its rows again; the other
            # cases run the backward on the mirror their forward filled
            with torch.no_grad():
                cp_attention(ql.detach() * 0, kl.detach() * 0, vl.detach() * 0, lay, plan, dist.group.WORLD, ex, Hq, Hkv)
        out.backward(do[idx])
        torch.cuda.synchronize()
        what = (f"cp ({'paired' if balance else 'contiguous'} pieces, {len(cu) - 1} documents, "
                f"{'tiles read from their owners' if direct else 'rows fetched once into the mirror'})")
        close(out, ref[idx], 2e-2, what + " out")
        close(ql.grad, qf.grad[idx], 3e-2, what + " dq")
        close(kl.grad, kf.grad[idx], 3e-2, what + " dk")
        close(vl.grad, vf.grad[idx], 3e-2, what + " dv")


def check_tensor_parallel_collectives(dev, rank, world):
    """Sequence gather and reduce-scatter over peer memory against NCCL, forward and backward."""
    from halo_b200.parallel.tensor_parallel import TensorParallel, gather_seq, reduce_scatter_seq

    T, H = 1024 * world, 256
    tp = TensorParallel(dist.group.WORLD, dev, hidden=H, max_tokens=T)
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    shard = torch.randn(T // world, H, device=dev, generator=g).bfloat16().requires_grad_()
    full = gather_seq(shard, tp)
    want = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(want, shard.detach())
    assert torch.equal(full, want), "tp gather"
    partial = torch.randn(T, H, device=dev, generator=g).bfloat16().requires_grad_()
    mine = reduce_scatter_seq(partial, tp)
    ref = partial.detach().float().clone()
    dist.all_reduce(ref)
    lo, hi = tp.shard_rows(T)
    close(mine, ref[lo:hi], 1e-2, "tp reduce-scatter")
    gy = torch.randn(T // world, H, device=dev, generator=g).bfloat16()
    mine.backward(gy)                                   # backward of a reduce-scatter is a gather
    want_g = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(want_g, gy)
    assert torch.equal(partial.grad, want_g), "tp reduce-scatter backward"
    full.backward(want_g)                               # backward of a gather is a reduce-scatter
    ref_g = want_g.float() * world
    close(shard.grad, ref_g[lo:hi], 1e-2, "tp gather backward")
    # the row-parallel product with the reduce-scatter's transfer in the GEMM epilogue
    from halo_b200.parallel.tensor_parallel import row_parallel_linear

    K = 384
    x = (torch.randn(T, K, device=dev, generator=g) * 0.1).bfloat16().requires_grad_()
    w = (torch.randn(H, K, device=dev, generator=g) * 0.1).bfloat16().requires_grad_()
    y = row_parallel_linear(x, w, tp)
    ref_y = x.detach().float() @ w.detach().float().t()
    dist.all_reduce(ref_y)
    close(y, ref_y[lo:hi], 2e-2, "tp fused gemm + reduce-scatter")
    y.backward(gy)
    close(x.grad, want_g.float() @ w.detach().float(), 2e-2, "tp row-parallel dx")
    close(w.grad, want_g.float().t() @ x.detach().float(), 2e-2, "tp row-parallel dw")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from halo_b200.ops import _lib
    from halo_b200.parallel.runtime import ParallelRuntime

    from halo_b200.parallel.runtime import SymmetricTransport

    parallel = ParallelRuntime.for_expert_parallel(world, dev)
    for fused in (True, False):
        tr = SymmetricTransport(dist.group.WORLD, dev)
        tr.fused = fused
        tr.configure(max_tokens=1536, top_k=4, hidden=512, n_local_experts=16 // world)
        check_expert_transport(tr, dev, rank, world, "movement inside the GEMM kernels" if fused else "separate push / pull kernels")
        _lib.raise_on_status(dev)
        if not fused:
            check_biased_glu_experts(tr, dev, rank, world)
            _lib.raise_on_status(dev)
    check_fused_optimizer(dev, rank, world)
    check_broadcast_and_allreduce(dev, rank, world)
    check_sharded_weight_push(dev, rank, world)
    check_zero3_layers(dev, rank, world)
    nvls = check_nvls_forms(dev, rank, world)
    check_context_parallel(dev, rank, world)
    check_tensor_parallel_collectives(dev, rank, world)
    _lib.raise_on_status(dev)
    dist.barrier()
    if rank == 0:
        print(f"CHECKS PASSED (world {world}; NVLS forms {'checked' if nvls else 'not available'})")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
