"""ZeRO-3 for the decoder layers: every layer's replicated matrices live as 1 / N slices on the N data-parallel ranks and
exist in full only while the layer runs.

What is sharded: the >= 2-D parameters of every decoder layer that are replicated today (attention projections, dense
feed-forward matrices, routers, shared experts; expert banks under expert parallelism and tensor-parallel slices already
are sharded and stay as they are). Embeddings, the head and the norm vectors stay replicated.

How a step runs (per-layer recomputation gives every layer exactly two windows in which its parameters are needed: its
first pass, and its re-run + backward):

* before a window the layer's slices are assembled into one of two local staging buffers by this rank's own pull kernel
  (16-byte loads from every peer's slice over NVLink), and the layer's parameters are pointed at views of that buffer;
  the NEXT layer's gather (the previous one in the backward pass) is issued at the same time on a side stream, so it runs
  under the current layer's compute and a layer never waits for its weights after the first;
* after the backward window the layer's full-size gradients (which autograd wrote straight into a symmetric staging
  buffer: the parameters' ``.grad`` are views of it) are reduced: a barrier, then every rank sums ITS slice over all
  ranks' buffers in fp32 (``rs_sum_norm_kernel``) and adds it to its fp32 gradient shard - the reduce-scatter of layer L
  runs while layer L - 1 computes;
* the optimizer steps one flat parameter per rank (``zero3_shard``: this rank's slices of every layer) with its fp32
  gradient shard; nothing is gathered after the step, the next forward pulls the new values.

Memory per rank: 1 / N of the layers' matrices (+ the same in fp32 gradients and the optimizer state) and two layers' worth
of staging for weights and for gradients.

On CPU (gloo tests) the gathers are ``all_gather_into_tensor`` and the reductions ``all_reduce`` + slice.

Counterpart of the reference's FSDP2 wrapping with ``reshard_after_forward`` (halo/distributed/fsdp.py:319-403, units of
decoder layers, mixed-precision policy :64-73); here without a wrapper around the modules: the model's own layer loop
calls ``before_layer`` / ``after_layer``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from halo_b200.ops import _lib

ALIGN = 8          # elements: 16 bytes of bf16


def _managed(p, ep_world: int) -> bool:
    if p.dim() < 2 or not p.requires_grad or getattr(p, "tp_kind", None) is not None:
        return False
    return not (getattr(p, "is_expert", False) and ep_world > 1)


class Zero3Layers:
    def __init__(self, model, group, device, ep_world: int = 1, prefetch: bool = True):
        self.model, self.group, self.device = model, group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.prefetch = prefetch and self.device.type == "cuda"
        self.layers = list(model.layers)
        self.params: list[list] = []          # per layer: (name, parameter, element offset in the layer's flat space, numel, shape)
        self.layer_len: list[int] = []        # per layer: flat elements, padded to world * ALIGN
        self.shard_off: list[int] = []        # per layer: element offset of the layer's slice inside this rank's flat shard
        dtype = None
        off = 0
        for li, layer in enumerate(self.layers):
            items, at = [], 0
            for name, p in layer.named_parameters():
                if not _managed(p, ep_world):
                    continue
                dtype = dtype or p.dtype
                if p.dtype != dtype:
                    raise ValueError(f"sharded layer parameters must share one dtype: {name} is {p.dtype}, others {dtype}")
                items.append((f"layers.{li}.{name}", p, at, p.numel(), tuple(p.shape)))
                at += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            unit = self.world * ALIGN
            total = (at + unit - 1) // unit * unit
            self.params.append(items)
            self.layer_len.append(total)
            self.shard_off.append(off)
            off += total // self.world
        if dtype is None:
            raise ValueError("the model has no layer parameters to shard")
        self.dtype = dtype
        self.shard_total = max(off, ALIGN)
        self.max_full = max(self.layer_len)
        cuda = self.device.type == "cuda"
        if cuda:
            import torch.distributed._symmetric_memory as symm

            if dtype != torch.bfloat16:
                raise ValueError("the GPU path shards bf16 parameters")
            shard = symm.empty((self.shard_total,), dtype=dtype, device=self.device)
            self.gstage = symm.empty((2, self.max_full), dtype=dtype, device=self.device)
            self.gstage.zero_()
            self._h_shard = symm.rendezvous(shard, group)
            self._h_g = symm.rendezvous(self.gstage, group)
            self._shard_ptrs = (_lib.c_void_p * self.world)(*list(self._h_shard.buffer_ptrs))
            self._g_ptrs = (_lib.c_void_p * self.world)(*list(self._h_g.buffer_ptrs))
            self.side = torch.cuda.Stream(device=self.device)
            n_blocks = int(_lib.lib().halo_rs_blocks(_lib.c_ll(self.max_full // self.world)))
            self._partial = torch.zeros(max(n_blocks, 1), dtype=torch.float32, device=self.device)
        else:
            shard = torch.empty(self.shard_total, dtype=dtype, device=self.device)
            self.gstage = torch.zeros((2, self.max_full), dtype=dtype, device=self.device)
            self.side = None
        self.stage = torch.zeros((2, self.max_full), dtype=dtype, device=self.device)
        self._tmp = torch.zeros(self.max_full // self.world, dtype=torch.float32, device=self.device)
        # this rank's slices of the initial values, then the full copies are dropped
        with torch.no_grad():
            shard.zero_()
            for li, items in enumerate(self.params):
                n = self.layer_len[li] // self.world
                lo, hi = self.rank * n, (self.rank + 1) * n
                dst = shard[self.shard_off[li]:self.shard_off[li] + n]
                for _, p, at, numel, _ in items:
                    a, b = max(at, lo), min(at + numel, hi)
                    if a < b:
                        dst[a - lo:b - lo].copy_(p.detach().reshape(-1)[a - at:b - at])
        self.shard = nn.Parameter(shard, requires_grad=True)
        self.shard.flat_matrices = True        # decays like the matrices it is made of, although it is 1-D
        self.shard.dp_sharded = True           # every rank holds different values: norms add over ranks, no gradient all-reduce
        self.grad_shard = torch.zeros(self.shard_total, dtype=torch.float32, device=self.device)
        if dtype != torch.float32:
            self.shard.grad_dtype = torch.float32      # a bf16 parameter with an fp32 gradient (the optimizer kernel takes both)
        self.shard.grad = self.grad_shard
        self._placeholder = torch.empty(0, dtype=dtype, device=self.device)
        for items in self.params:
            for _, p, *_ in items:
                p.data = self._placeholder
                p.zero3_managed = True
        self._ready = [None, None]            # event after which stage[slot] holds _slot_layer[slot]
        self._slot_layer = [-1, -1]
        self._free = [None, None]             # event after which stage[slot] may be overwritten
        self._grads_pending = False
        model.zero3_shard = self.shard         # registered: optimizers and state dicts see it
        model.layer_hooks = self
        model.zero3 = self
        self.barrier()

    # ---- plumbing ---------------------------------------------------------------------------------------
    def barrier(self) -> None:
        if self.device.type == "cuda":
            self._h_shard.barrier(channel=5)
        elif self.world > 1:
            dist.barrier(group=self.group)

    def _gather_into(self, li: int, slot: int, stream=None) -> None:
        n = self.layer_len[li] // self.world
        dst = self.stage[slot, :self.layer_len[li]]
        if self.device.type == "cuda":
            esize = self.shard.element_size()
            rc = _lib.lib().halo_allgather_pull(_lib.ptr(dst), self._shard_ptrs, _lib.c_int(self.world),
                                                _lib.c_ll(self.shard_off[li] * esize), _lib.c_ll(n * esize),
                                                _lib.c_void_p(stream.cuda_stream) if stream is not None else _lib.stream_ptr(self.device))
            _lib.check(rc, "halo_allgather_pull")
        else:
            mine = self.shard.data[self.shard_off[li]:self.shard_off[li] + n].contiguous()
            if self.world > 1:
                dist.all_gather_into_tensor(dst, mine, group=self.group)
            else:
                dst.copy_(mine)

    def _issue_gather(self, li: int) -> int:
        """Start assembling layer ``li`` in its slot (on the side stream when prefetching). Returns the slot."""
        slot = li % 2
        if self._slot_layer[slot] == li:
            return slot
        if self.device.type == "cuda":
            main = torch.cuda.current_stream(self.device)
            stream = self.side if self.prefetch else main
            if self._free[slot] is not None:
                stream.wait_event(self._free[slot])       # the layer that used this slot is done with it
            if stream is not main:
                ev0 = torch.cuda.Event()
                ev0.record(main)
                stream.wait_event(ev0)                    # and nothing issued earlier can still be writing the shard
            self._gather_into(li, slot, stream)
            ev = torch.cuda.Event()
            ev.record(stream)
            self._ready[slot] = ev
        else:
            self._gather_into(li, slot)
        self._slot_layer[slot] = li
        return slot

    def _bind(self, li: int, slot: int, with_grads: bool) -> None:
        flat = self.stage[slot]
        for _, p, at, numel, shape in self.params[li]:
            p.data = flat[at:at + numel].view(shape)
            if with_grads:
                p.grad = self.gstage[slot, at:at + numel].view(shape)

    def _unbind(self, li: int) -> None:
        for _, p, *_ in self.params[li]:
            p.data = self._placeholder
            p.grad = None

    # ---- the hooks the layer loop calls --------------------------------------------------------------------
    def before_layer(self, li: int, backward: bool) -> None:
        slot = self._issue_gather(li)
        nxt = li - 1 if backward else li + 1
        if self.device.type == "cuda":
            if self._ready[slot] is not None:
                torch.cuda.current_stream(self.device).wait_event(self._ready[slot])
            if self.prefetch and 0 <= nxt < len(self.layers):
                self._issue_gather(nxt)                   # runs under this layer's compute
        if backward:
            self.gstage[slot, :self.layer_len[li]].zero_()
        self._bind(li, slot, with_grads=backward)

    def after_layer(self, li: int, backward: bool) -> None:
        slot = li % 2
        self._unbind(li)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._free[slot] = ev
        if backward:
            self._reduce_scatter(li, slot)

    def _reduce_scatter(self, li: int, slot: int) -> None:
        n = self.layer_len[li] // self.world
        dst = self.grad_shard[self.shard_off[li]:self.shard_off[li] + n]
        if self.device.type == "cuda":
            self._h_g.barrier(channel=6)                   # every rank's gradients of this layer are written
            lo = slot * self.max_full + self.rank * n
            rc = _lib.lib().halo_rs_sum_norm(self._g_ptrs, _lib.c_int(self.world), _lib.c_ll(lo), _lib.c_ll(n),
                                             _lib.ptr(self._tmp), _lib.ptr(self._partial), _lib.stream_ptr(self.device))
            _lib.check(rc, "halo_rs_sum_norm")
            dst.add_(self._tmp[:n])
            # peers may still be reading this slot: it is zeroed again two layers later, after that layer's barrier,
            # which no rank passes before its own reduction of this layer was issued
        else:
            full = self.gstage[slot, :self.layer_len[li]].float()
            if self.world > 1:
                dist.all_reduce(full, group=self.group)
            dst.add_(full[self.rank * n:(self.rank + 1) * n])
        self._grads_pending = True

    # ---- around the optimizer -------------------------------------------------------------------------------
    def before_step(self) -> None:
        """COLLECTIVE: no peer reads this rank's slices any more (the last gather of the backward pass is done everywhere)."""
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).wait_stream(self.side)
        self.barrier()

    def after_step(self) -> None:
        """COLLECTIVE: every rank's slices hold the new values; staged copies are stale."""
        self._slot_layer = [-1, -1]
        self.grad_shard.zero_()
        self.shard.grad = self.grad_shard
        self._grads_pending = False
        self.barrier()

    # ---- whole tensors (saving, inspection) -------------------------------------------------------------------
    def full_tensors(self, li: int) -> dict:
        """COLLECTIVE: ``{name inside the model: full tensor}`` of layer ``li`` (fresh copies)."""
        flat = torch.empty(self.layer_len[li], dtype=self.dtype, device=self.device)
        n = self.layer_len[li] // self.world
        mine = self.shard.data[self.shard_off[li]:self.shard_off[li] + n].contiguous()
        if self.world > 1:
            dist.all_gather_into_tensor(flat, mine, group=self.group)
        else:
            flat.copy_(mine)
        return {name: flat[at:at + numel].view(shape).clone() for name, _, at, numel, shape in self.params[li]}

    def managed_names(self) -> set:
        return {name for items in self.params for name, *_ in items}

    def load_full(self, named: dict) -> None:
        """Take this rank's slices out of full tensors (``{name: tensor}``, e.g. from a checkpoint)."""
        with torch.no_grad():
            for li, items in enumerate(self.params):
                n = self.layer_len[li] // self.world
                lo, hi = self.rank * n, (self.rank + 1) * n
                dst = self.shard.data[self.shard_off[li]:self.shard_off[li] + n]
                for name, _, at, numel, _ in items:
                    a, b = max(at, lo), min(at + numel, hi)
                    if a < b:
                        dst[a - lo:b - lo].copy_(named[name].reshape(-1)[a - at:b - at].to(dst.dtype))
        self._slot_layer = [-1, -1]
        self.barrier()


def shard_layers(model, group, device, ep_world: int = 1) -> Zero3Layers:
    """Shard ``model``'s decoder-layer matrices over ``group`` (see the module docstring). Call after the weights are
    loaded and before the optimizer is built."""
    for layer in model.layers:
        layer.recompute_policy = "full"
    return Zero3Layers(model, group, device, ep_world)
