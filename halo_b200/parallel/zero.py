"""Sharded AdamWBF16 for the replicated parameters, fused with its collectives.

The replicated (non-expert) bf16 parameters of a data-parallel group live in one flat buffer per
rank, allocated as symmetric memory so every rank can address every peer's copy; so does a flat
gradient buffer. Each rank owns one contiguous slice of the flat space and the bf16 moments of
that slice only (optimizer state is sharded N ways). One optimizer step is

  (backward) every parameter's ``.grad`` IS its range of the flat gradient buffer, so autograd
             accumulates straight into it; a gradient found elsewhere is copied in       (local)
  barrier
  reduce     the owner sums its slice over all peers' buffers in fp32 and     (peer loads)
             gets the slice's contribution to the global gradient norm
  [the caller combines the norm pieces and derives the clip coefficient]
  update     AdamWBF16 on the slice; the new bf16 weights are stored into     (peer stores)
             every peer's parameter buffer, which is the all-gather
  barrier

so reduce-scatter, cast / scale, optimizer and all-gather are two kernels that move each gradient
and each weight across NVLink exactly once, instead of NCCL reduce-scatter + a local optimizer +
NCCL all-gather. Arithmetic and rounding noise equal the unsharded optimizer's (the noise is keyed
by parameter name and element offset, not by the sharding).

Counterpart of FSDP2's post-backward reduce-scatter + the reference's AdamWBF16 + the next
unshard (halo/distributed/fsdp.py:319-403, halo/optimizers/adamw_bf16.py:378-499).
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch
import torch.distributed as dist

from halo_b200.ops import _lib
from halo_b200.optim.adamw_bf16 import SR_KEY, param_name_hash


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FusedShardedAdamW:
    def __init__(self, named_params, group, device, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 key: int = SR_KEY, replicate_group=None, nvls: bool | None = None):
        """``group``: the ranks the flat space is cut over (the ``dp_shard`` axis). ``replicate_group``: under hybrid
        sharding, the ranks that own the SAME slice in the other shard groups (the ``dp_replicate`` axis); every owner
        adds its peers' slice sums before the update, so all copies of a slice take the same step."""
        import torch.distributed._symmetric_memory as symm

        # NVLS: reduce through multimem.ld_reduce and all-gather through multimem.st when the buffers are bound to an
        # NVLink multicast object. The in-switch reduction delivers bf16-rounded sums (as a bf16 all-reduce does), so
        # this mode is not bit-identical to the unsharded optimizer; it is off unless asked for (HALO_ZERO_NVLS=1).
        from halo_b200 import env

        self._want_nvls = env.zero_nvls() if nvls is None else bool(nvls)
        self.replicate_group = replicate_group
        self.n_replicas = dist.get_world_size(replicate_group) if replicate_group is not None else 1
        self.group, self.device = group, torch.device(device)
        self.n_ranks, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.lr, self.betas, self.eps, self.weight_decay, self.key = lr, betas, eps, weight_decay, key
        self.step_count = 0
        self.named = [(n, p) for n, p in named_params if p.requires_grad]
        for n, p in self.named:
            if p.dtype != torch.bfloat16:
                raise TypeError(f"{n}: the fused sharded optimizer takes bf16 parameters")
        # flat layout: every tensor starts on a multiple of 8 elements
        self.offsets, off = [], 0
        for _, p in self.named:
            self.offsets.append(off)
            off += _round_up(p.numel(), 8)
        self.total = _round_up(max(off, 8), 8 * self.n_ranks)
        self.shard = self.total // self.n_ranks
        self.lo = self.rank * self.shard
        self.flat_p = symm.empty((self.total,), dtype=torch.bfloat16, device=self.device)
        self.flat_g = symm.empty((self.total,), dtype=torch.bfloat16, device=self.device)
        self.flat_p.zero_()
        self.flat_g.zero_()
        self.hp = symm.rendezvous(self.flat_p, group)
        self.hg = symm.rendezvous(self.flat_g, group)
        with torch.no_grad():
            for (n, p), o in zip(self.named, self.offsets):
                view = self.flat_p[o:o + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view            # the model now reads the flat buffer directly
        self.m = torch.zeros(self.shard, dtype=torch.bfloat16, device=self.device)
        self.v = torch.zeros(self.shard, dtype=torch.bfloat16, device=self.device)
        self.gsum = torch.empty(self.shard, dtype=torch.float32, device=self.device)
        L = _lib.lib()
        self.rs_blocks = int(L.halo_rs_blocks(_lib.c_ll(self.shard)))
        self.partial = torch.zeros(self.rs_blocks, dtype=torch.float32, device=self.device)
        self.shard_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._build_segments()
        self._p_ptrs = (_lib.c_void_p * self.n_ranks)(*list(self.hp.buffer_ptrs))
        self._g_ptrs = (_lib.c_void_p * self.n_ranks)(*list(self.hg.buffer_ptrs))
        mc_p, mc_g = int(getattr(self.hp, "multicast_ptr", 0) or 0), int(getattr(self.hg, "multicast_ptr", 0) or 0)
        self.nvls = bool(self._want_nvls and mc_p and mc_g and self.n_ranks > 1)
        self._mc_p, self._mc_g = (mc_p, mc_g) if self.nvls else (0, 0)
        self._grad_views = [self.flat_g[o:o + p.numel()].view(p.shape) for (_, p), o in zip(self.named, self.offsets)]
        self._attach_grad_views()
        self.hp.barrier(channel=0)

    def _attach_grad_views(self) -> None:
        """Point every parameter's ``.grad`` at its range of the (zeroed) flat gradient buffer. Autograd adds into an
        existing ``.grad`` in place, so the backward writes the buffer the reduce kernel reads: no packing pass."""
        for (_, p), view in zip(self.named, self._grad_views):
            p.grad = view

    def _build_segments(self) -> None:
        L = _lib.lib()
        epb = int(L.halo_slice_elems_per_block())
        lo, hi = self.lo, self.lo + self.shard
        seg_off, seg_len, seg_toff, seg_hash, seg_wd, blocks = [], [], [], [], [], [0]
        for (n, p), o in zip(self.named, self.offsets):
            a, b = max(lo, o), min(hi, o + _round_up(p.numel(), 8))
            if a >= b:
                continue
            seg_off.append(a - lo)
            seg_len.append(b - a)
            seg_toff.append(a - o)
            seg_hash.append(param_name_hash(n))
            seg_wd.append(self.weight_decay if p.dim() > 1 else 0.0)
            blocks.append(blocks[-1] + (b - a + epb - 1) // epb)
        dev = self.device
        self.n_seg, self.total_blocks = len(seg_off), blocks[-1]
        self.seg_off = torch.tensor(seg_off, dtype=torch.int64, device=dev)
        self.seg_len = torch.tensor(seg_len, dtype=torch.int64, device=dev)
        self.seg_toff = torch.tensor(seg_toff, dtype=torch.int64, device=dev)
        self.seg_hash = torch.from_numpy(np.asarray(seg_hash, dtype=np.uint64).view(np.int64)).to(dev)
        self._seg_decay = seg_wd
        self._seg_decay_dev = torch.tensor(seg_wd or [0.0], dtype=torch.float64, device=dev)
        self.seg_wd = torch.ones(max(1, len(seg_wd)), dtype=torch.float32, device=dev)
        self.block_start = torch.tensor(blocks, dtype=torch.int32, device=dev)

    # ---- step phases ---------------------------------------------------------------------------
    @torch.no_grad()
    def pack_and_reduce(self) -> torch.Tensor:
        """Phase 1. Returns the device scalar ``sum of squares`` of this rank's slice of the summed gradient."""
        for (n, p), view in zip(self.named, self._grad_views):
            g = p.grad
            if g is None:
                view.zero_()                      # someone dropped the gradient: this parameter contributes nothing
            elif g.data_ptr() != view.data_ptr():
                view.copy_(g)                     # a gradient that was replaced instead of accumulated in place
        self.hg.barrier(channel=0)
        L = _lib.lib()
        s = _lib.stream_ptr(self.device)
        if self.nvls:
            _lib.check(L.halo_rs_sum_norm_mc(_lib.c_void_p(self._mc_g), _lib.c_ll(self.lo), _lib.c_ll(self.shard),
                                             _lib.ptr(self.gsum), _lib.ptr(self.partial), s), "halo_rs_sum_norm_mc")
        else:
            _lib.check(L.halo_rs_sum_norm(self._g_ptrs, _lib.c_int(self.n_ranks), _lib.c_ll(self.lo), _lib.c_ll(self.shard),
                                          _lib.ptr(self.gsum), _lib.ptr(self.partial), s), "halo_rs_sum_norm")
        if self.n_replicas > 1:
            # hybrid sharding: the slice's sum over the other shard groups (fp32, one library all-reduce of 1/N of the
            # gradient), and its norm from the completed sum. Every replica of a slice reports the same square, so each
            # reports its share: the caller's sum over all ranks then counts the slice once.
            dist.all_reduce(self.gsum, group=self.replicate_group)
            self.shard_sq.copy_((self.gsum.double().pow(2).sum() / self.n_replicas).float().reshape(1))
        else:
            self.shard_sq.copy_(self.partial.sum().reshape(1))
        return self.shard_sq

    @torch.no_grad()
    def step(self, grad_scale: torch.Tensor | None = None, skip: torch.Tensor | None = None) -> None:
        """Phase 2 (after the caller has turned the norm pieces into ``grad_scale`` / ``skip``)."""
        self.step_count += 1
        b1, b2 = self.betas
        t = self.step_count
        step_size = self.lr / (1.0 - b1**t)
        bc2_sqrt = math.sqrt(1.0 - b2**t)
        # 1 - lr * decay per segment, formed on the device in double and rounded once to fp32 (what the unsharded
        # optimizer's host-side double arithmetic gives)
        self.seg_wd.copy_(torch.mul(self._seg_decay_dev, -float(self.lr)).add_(1.0))
        L = _lib.lib()
        rc = L.halo_adam_allgather(
            self._p_ptrs, _lib.c_int(self.n_ranks), _lib.c_int(self.rank), _lib.c_ll(self.lo), _lib.ptr(self.gsum),
            _lib.ptr(self.m), _lib.ptr(self.v), _lib.ptr(self.seg_off), _lib.ptr(self.seg_len), _lib.ptr(self.seg_toff),
            _lib.ptr(self.seg_hash), _lib.ptr(self.seg_wd), _lib.ptr(self.block_start), _lib.c_int(self.n_seg),
            _lib.c_int(self.total_blocks), _lib.c_float(b1), _lib.c_float(b2), _lib.c_float(step_size),
            _lib.c_float(bc2_sqrt), _lib.c_float(self.eps), ctypes.c_ulonglong(self.key), ctypes.c_ulonglong(t),
            _lib.ptr(grad_scale), _lib.ptr(skip), _lib.stream_ptr(self.device), _lib.c_void_p(self._mc_p),
        )
        _lib.check(rc, "halo_adam_allgather")
        self.hp.barrier(channel=0)

    def zero_grad(self) -> None:
        """One fill of the flat gradient buffer; the parameters keep (or get back) their views into it."""
        self.flat_g.zero_()
        self._attach_grad_views()

    # ---- bookkeeping ---------------------------------------------------------------------------
    def bytes_over_nvlink_per_step(self) -> int:
        """Gradient slice read from N-1 peers + weight slice stored to N-1 peers (bf16)."""
        return 2 * 2 * self.shard * (self.n_ranks - 1)

    def state_dict(self) -> dict:
        return {"step": self.step_count, "m": self.m.cpu(), "v": self.v.cpu(), "lo": self.lo, "shard": self.shard,
                "n_ranks": self.n_ranks, "n_replicas": self.n_replicas}

    def load_state_dict(self, sd: dict) -> None:
        if sd["n_ranks"] != self.n_ranks or sd["shard"] != self.shard:
            raise ValueError("the sharded optimizer state was saved under a different data-parallel width")
        self.step_count = sd["step"]
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])


class NoParametersLeft:
    """Stands in for the ordinary optimizer when every parameter went to the fused sharded optimizer (a dense
    model): it accepts the engine's calls and owns the learning-rate slot the scheduler writes."""

    def __init__(self, lr: float):
        self.param_groups = [{"lr": lr, "params": []}]
        self.state: dict = {}

    def defer_grad_scale(self, scale) -> None: ...
    def arm_skip(self, flag) -> None: ...
    def step(self) -> None: ...
    def zero_grad(self, set_to_none: bool = True) -> None: ...

    def state_dict(self) -> dict:
        return {"param_groups": [{"lr": self.param_groups[0]["lr"]}]}

    def load_state_dict(self, sd: dict) -> None:
        self.param_groups[0]["lr"] = sd["param_groups"][0]["lr"]
