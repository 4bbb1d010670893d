"""Run-time side of the parallel layout on one NVLink/NVSwitch box: the expert-parallel transport
over peer-mapped (symmetric) memory and the gradient synchronisation of the replicated parameters.

``SymmetricTransport`` gives the MoE kernels what they need to move tokens themselves: one set of
row buffers per rank, allocated once through ``torch.distributed._symmetric_memory`` so that every
rank holds a device pointer to every peer's buffer, plus a device-side barrier between the push,
compute and pull phases. The kernels then store to / load from peer memory directly; no collective
library call carries token data.

``ParallelRuntime`` owns the groups of a run and the per-step reductions: replicated (non-expert)
gradients are summed over the data-parallel group, expert gradients over the expert-replica group
when experts are replicated, and the global gradient norm is assembled from the pieces each group
tiles exactly once.

Counterpart of the reference's EP config / dispatcher plumbing and gradient sweeps
(halo/distributed/expert_parallel/config.py:149-280, halo/trainers/parallelism/grad_sync.py:159-210,
halo/trainers/parallelism/grad_clipping.py:161-228).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from halo_b200.ops import _lib


class SymmetricTransport:
    """Expert-parallel transport over peer-mapped buffers of one process group."""

    def __init__(self, group, device, capacity_factor: float = 1.5, n_lanes: int = 1, channel_base: int = 0):
        """``n_lanes`` > 1: the tokens of one MoE call are cut into that many parts, each routed through its own
        half-size buffers on its own stream, so one part's transfers over NVLink run beside another part's expert
        products. ``channel_base``: first barrier channel of this transport (three are used)."""
        self.group = group
        self.channel_base = channel_base
        self.lanes = ([SymmetricTransport(group, device, capacity_factor, 1, 4 * (i + 1)) for i in range(n_lanes)]
                      if n_lanes > 1 else None)
        self.stream = None
        self.device = torch.device(device)
        self.n_ranks = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.capacity_factor = capacity_factor
        self._bufs: dict[str, tuple[torch.Tensor, object]] = {}
        self._cap = None
        self._hidden = None
        self._barrier_handle = None
        self._side = None
        self.stable_until_backward = True
        # fused path: dispatch inside the first expert GEMM, combine inside the last one's epilogue, counts exchanged
        # through peer memory (halo_b200/csrc/moe_fused_sm100.cu)
        from halo_b200 import env

        self.fused = env.moe_fused()
        self.seq = 0                      # calls made through the control block (every rank counts alike)
        self.max_tiles = 0
        self.n_experts = 0

    # ---- provisioning ---------------------------------------------------------------------
    def configure(self, max_tokens: int, top_k: int, hidden: int, n_local_experts: int) -> None:
        """Allocate the row buffers for the largest batch this run will route (collective call)."""
        import torch.distributed._symmetric_memory as symm

        if self.lanes:
            per_lane = ((max_tokens + len(self.lanes) - 1) // len(self.lanes) + 127) // 128 * 128
            for lane in self.lanes:
                lane.configure(per_lane, top_k, hidden, n_local_experts)
                lane.stream = torch.cuda.Stream(device=self.device)
            return
        mean_rows = max_tokens * top_k  # every rank sends max_tokens * top_k slots; on average it receives as many
        cap = int(self.capacity_factor * mean_rows) + 128 * n_local_experts
        cap = (cap + 127) // 128 * 128
        self._cap, self._hidden = cap, hidden
        slots = max_tokens * top_k
        if self.fused:
            self.n_experts = n_local_experts * self.n_ranks
            self.max_tiles = cap // 128
            ctrl_ints = 2 * self.n_ranks * self.n_experts + self.n_ranks + 2 * self.max_tiles
            specs = (("recv_x", cap, hidden, torch.bfloat16), ("recv_dy", cap, hidden, torch.bfloat16),
                     ("slots", slots, hidden, torch.bfloat16), ("row_w", cap, 1, torch.float32),
                     ("row_meta", cap, 1, torch.int32), ("dw_slots", slots, 1, torch.float32),
                     ("ctrl", ctrl_ints, 1, torch.int32))
        else:
            specs = (("recv_x", cap, hidden, torch.bfloat16), ("y_rows", cap, hidden, torch.bfloat16),
                     ("recv_dy", cap, hidden, torch.bfloat16), ("dx_rows", cap, hidden, torch.bfloat16),
                     ("row_w", cap, 1, torch.float32), ("dwrow", cap, 1, torch.float32))
        for name, rows, cols, dtype in specs:
            t = symm.empty((rows, cols), dtype=dtype, device=self.device)
            if name == "ctrl":
                t.zero_()
            hdl = symm.rendezvous(t, self.group)
            if int(getattr(hdl, "world_size", self.n_ranks)) != self.n_ranks or int(getattr(hdl, "rank", self.rank)) != self.rank:
                # the peer table must be this group's: kernels index it by the group rank
                raise RuntimeError(f"symmetric-memory handle of {name!r} describes rank {hdl.rank} of {hdl.world_size}, the "
                                   f"expert-parallel group has rank {self.rank} of {self.n_ranks}")
            self._bufs[name] = (t, hdl)
        self._barrier_handle = self._bufs["recv_x"][1]
        if self.fused:
            torch.cuda.synchronize(self.device)
            self._barrier_handle.barrier(channel=self.channel_base)      # every rank's control block is zero before the first call
            self.seq = 0

    def capacity(self, n_slots: int, n_local_experts: int) -> int:
        if self._cap is None:
            raise RuntimeError("SymmetricTransport.configure() must run before the first MoE layer")
        return self._cap

    def buffer(self, name: str, rows: int, cols: int, dtype: torch.dtype, device) -> torch.Tensor:
        t, _ = self._bufs[name]
        if t.shape[0] < rows or t.shape[1] != cols or t.dtype != dtype:
            raise RuntimeError(f"symmetric buffer {name!r} {tuple(t.shape)} cannot serve [{rows}, {cols}] {dtype}")
        return t

    def peer_table(self, buf: torch.Tensor):
        for t, hdl in self._bufs.values():
            if t.data_ptr() == buf.data_ptr():
                ptrs = list(hdl.buffer_ptrs)
                return (_lib.c_void_p * self.n_ranks)(*ptrs)
        raise RuntimeError("peer_table() needs a buffer handed out by this transport")

    # ---- control block of the fused path ------------------------------------------------------
    def next_seq(self) -> int:
        """Number of the next call through the control block (1, 2, ...): flag value and buffer parity of that call."""
        self.seq += 1
        return self.seq

    def ctrl_table(self):
        return self.peer_table(self._bufs["ctrl"][0])

    def arrive_table(self, seq: int):
        """Every rank's arrival counters of the call ``seq`` (the control block's second half, by parity)."""
        off = 4 * (2 * self.n_ranks * self.n_experts + self.n_ranks + (seq & 1) * self.max_tiles)
        ptrs = [p + off for p in self._bufs["ctrl"][1].buffer_ptrs]
        return (_lib.c_void_p * self.n_ranks)(*ptrs)

    # ---- control plane -----------------------------------------------------------------------
    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """All ranks' per-expert slot counts, ``[n_ranks, E]`` (tiny; NCCL all-gather)."""
        out = torch.empty((self.n_ranks, counts.numel()), dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(out, counts.contiguous(), group=self.group)
        return out

    def barrier(self, channel: int = 0) -> None:
        """Device-side barrier on the current stream: peer stores issued before it are visible to
        peer loads issued after it. Bounded by the symmetric-memory barrier's own timeout. Barriers issued
        from different streams use different channels, so that their arrivals cannot pair up crosswise."""
        self._barrier_handle.barrier(channel=self.channel_base + channel)

    def barrier_before_push(self) -> None:
        """Run before an expert op fills peers' receive buffers: every rank has finished the products of its
        previous expert op that still read those buffers (they may run beside that op's pull on another stream)."""
        self._barrier_handle.barrier(channel=self.channel_base + 2)

    def side_stream(self, device):
        if self._side is None:
            self._side = torch.cuda.Stream(device=device)
        return self._side

    @property
    def transient_buffers(self) -> bool:
        # the buffers are reused by the next MoE layer; with per-layer recomputation the backward of a
        # layer runs right after its own forward, so they are still intact then
        return not self.stable_until_backward

    def reference_ffn(self, x, topk_idx, topk_w, w_gate_up, w_down):
        raise RuntimeError("the CPU expert-parallel path uses GlooTransport (halo_b200.parallel.expert_parallel)")


class ParallelRuntime:
    """Groups and per-step reductions of one run."""

    def __init__(self, device, dp_group=None, ep_group=None, expert_replica_group=None, transport=None,
                 tensor_parallel=None, context_parallel=None, tp_replica_group=None):
        """``dp_group``: every rank that holds a copy of the replicated parameters and sees its own tokens (data,
        context and tensor-parallel ranks alike: all three cut the tokens). ``tensor_parallel`` /
        ``context_parallel``: the objects the model carries when those axes are on. ``tp_replica_group``: ranks
        with the same tensor-parallel rank (they hold the same weight slices); None when tp spans the job."""
        self.device = torch.device(device)
        self.tensor_parallel = tensor_parallel
        self.context_parallel = context_parallel
        self.tp_replica_group = tp_replica_group
        self.dp_group = dp_group
        self.ep_group = ep_group
        self.expert_replica_group = expert_replica_group
        self.transport = transport
        self.dp_world = dist.get_world_size(dp_group) if dp_group is not None else 1
        self.ep_world = dist.get_world_size(ep_group) if ep_group is not None else 1
        self._flat = None
        self.fused_optimizer = None   # halo_b200.parallel.zero.FusedShardedAdamW for the replicated parameters

    def enable_fused_optimizer(self, model, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, dp_replicate_size: int = 1):
        """Shard the optimizer of the replicated parameters over the data-parallel group and fuse it
        with its reduce-scatter / all-gather. Returns the (name, parameter) pairs the caller still has to
        give an ordinary optimizer: the experts. ``dp_replicate_size > 1`` is hybrid sharding: the data-parallel ranks
        form that many replica groups (a ``(dp_replicate, dp_shard)`` mesh over the whole job); state is cut inside a
        group, and owners of the same slice add their sums across groups."""
        from halo_b200.parallel.zero import FusedShardedAdamW

        shared = [(n, p) for n, p in model.named_parameters() if not getattr(p, "is_expert", False)]
        experts = [(n, p) for n, p in model.named_parameters() if getattr(p, "is_expert", False)]
        shard_group, replicate_group = self.dp_group, None
        if dp_replicate_size > 1:
            from halo_b200.parallel.mesh import build_dp_mesh, shard_and_replicate_groups

            self.dp_mesh = build_dp_mesh(self.dp_world, dp_replicate_size, device_type=self.device.type)
            shard_group, replicate_group = shard_and_replicate_groups(self.dp_mesh)
        self.fused_optimizer = FusedShardedAdamW(shared, shard_group, self.device, lr, betas, eps, weight_decay,
                                                 replicate_group=replicate_group)
        return experts

    @classmethod
    def for_expert_parallel(cls, world: int, device, group=None, n_lanes: int = 1) -> "ParallelRuntime":
        """EP over every rank of ``group`` (default: the job); the non-expert parameters are replicated
        over the same ranks."""
        group = group if group is not None else dist.group.WORLD
        transport = SymmetricTransport(group, device, n_lanes=n_lanes)
        return cls(device, dp_group=group, ep_group=group, expert_replica_group=None, transport=transport)

    # ---- scalars -----------------------------------------------------------------------------
    def sum_scalar_over_dp(self, value: float) -> torch.Tensor:
        t = torch.tensor([value], dtype=torch.float32, device=self.device)
        dist.all_reduce(t, group=self.dp_group)
        return t.clamp_min(1.0)

    # ---- gradients ---------------------------------------------------------------------------
    def split_params(self, model):
        """(expert-sharded, replicated) parameters that have a gradient; tensor-parallel slices are a third
        kind, returned by :meth:`sliced_params`. Without expert parallelism the expert banks are replicated like
        everything else."""
        experts, shared = [], []
        for p in model.parameters():
            if p.grad is None or getattr(p, "tp_kind", None) is not None or getattr(p, "dp_sharded", False):
                continue
            (experts if getattr(p, "is_expert", False) and self.ep_world > 1 else shared).append(p)
        return experts, shared

    @staticmethod
    def dp_sharded_params(model):
        """Parameters of which every data-parallel rank holds a different 1 / N (a ZeRO-3 flat shard): their gradients are
        already reduced, their squared norms add over the ranks."""
        return [p for p in model.parameters() if p.grad is not None and getattr(p, "dp_sharded", False)]

    @staticmethod
    def sliced_params(model):
        return [p for p in model.parameters() if p.grad is not None and getattr(p, "tp_kind", None) is not None]

    def slice_batch(self, batch):
        """This rank's part of a packed row under context or tensor parallelism (both cut the tokens; positions and
        document boundaries of the whole row stay available to attention)."""
        from halo_b200.data.packing import PackedBatch
        from halo_b200.parallel.context_parallel import chunk_bounds

        if self.context_parallel is not None:
            from halo_b200.parallel.context_parallel import slice_batch

            return slice_batch(batch, self.context_parallel.rank, self.context_parallel.size, self.context_parallel.balance)
        if self.tensor_parallel is not None:
            tp = self.tensor_parallel
            lo, hi = chunk_bounds(batch.n_tokens, tp.size, tp.rank)
            labels = batch.labels[lo:hi]
            return PackedBatch(batch.input_ids[lo:hi], batch.position_ids, labels, batch.cu_seqlens,
                               int((labels != -100).sum()))
        return batch

    def sync_gradients(self, model) -> None:
        """Sum the replicated parameters' gradients over the data-parallel group (the loss is already
        normalised by the global token count, so a sum is the average the optimizer wants)."""
        experts, shared = self.split_params(model)
        if self.dp_world > 1 and shared:
            by_dtype: dict[torch.dtype, list] = {}
            for p in shared:
                by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
            for grads in by_dtype.values():
                flat = torch.cat([g.reshape(-1) for g in grads])
                dist.all_reduce(flat, group=self.dp_group)
                off = 0
                for g in grads:
                    n = g.numel()
                    g.copy_(flat[off:off + n].view_as(g))
                    off += n
        if self.expert_replica_group is not None and experts:
            for p in experts:
                dist.all_reduce(p.grad, group=self.expert_replica_group)
        if self.tp_replica_group is not None:
            for p in self.sliced_params(model):       # a slice saw every token of its replica's rows already
                dist.all_reduce(p.grad, group=self.tp_replica_group)

    def global_grad_sq_norm(self, model, grad_norm) -> None:
        """total_sq = ||replicated grads||^2 (counted once) + sum over EP ranks of ||expert grads||^2."""
        experts, shared = self.split_params(model)
        grad_norm.accumulate([p.grad for p in experts], first=True)
        if self.ep_world > 1:
            dist.all_reduce(grad_norm.total_sq, group=self.ep_group)
        sliced = self.sliced_params(model)
        if sliced:
            # every tensor-parallel rank holds a different slice: sum their squares over the tensor-parallel group
            tmp = grad_norm.total_sq.clone()
            grad_norm.accumulate([p.grad for p in sliced], first=True)
            dist.all_reduce(grad_norm.total_sq, group=self.tensor_parallel.group)
            grad_norm.total_sq.add_(tmp)
        sharded = self.dp_sharded_params(model)
        if sharded:
            tmp = grad_norm.total_sq.clone()
            grad_norm.accumulate([p.grad for p in sharded], first=True)
            if self.dp_world > 1:
                dist.all_reduce(grad_norm.total_sq, group=self.dp_group)
            grad_norm.total_sq.add_(tmp)
        grad_norm.accumulate([p.grad for p in shared], first=False)
