"""Context parallelism on packed rows: the row is cut into pieces, every rank owns some of them; everything except
attention is token-local; attention needs, for every query a rank owns, the keys and values of the earlier tokens of the
same document, which may live on other ranks.

**Layout.** With ``balance`` (the default) the row is cut into ``2 * cp`` pieces and rank ``r`` owns pieces ``r`` and
``2 cp - 1 - r`` (one early, one late): under a causal mask the attention work of a long document is then the same on
every rank, where contiguous chunks would give the last rank ``2 cp - 1`` times the work of the first. Piece boundaries
that fall inside a document are moved to the nearest multiple of 128 tokens from the document's start, so no 128-row
attention tile ever straddles two owners; ranks may therefore hold slightly different token counts (the loss is
normalised by the global count, expert dispatch exchanges per-rank counts anyway).

**Exchange (GPU).** Each rank publishes its keys and values (after rotary) in a symmetric buffer. The flash kernels
work in the row's global coordinates (masks, document ends, tile starts); queries, outputs and statistics are addressed
in the rank's local order, so no zero-padded query tensor exists. Keys and values come from a local mirror indexed by
global row that is filled once per exchange: the rank's own rows and exactly the foreign rows its queries can see, each
pulled over NVLink once by the rank's own copy kernel. (The kernels can instead read every foreign tile from its owner
through per-rank tensor maps; that was measured: fine for chat-length documents, five times slower than the mirror on
one 64k-token document, where every CTA's read of a tile crosses the link again.) In the backward pass dK / dV are
written at their global rows into a staging buffer; each owner takes its own rows and adds the peers' contributions in
rank order (deterministic, no atomics). Under per-layer recomputation the backward pass reuses the mirror its own
forward has just filled and exchanges nothing but the gradients.

The reference's context parallelism is Ulysses all-to-all and refuses packed rows
(halo/distributed/context_parallel/ulysses_model.py:199-312, model_rules.py); this is the packed-row replacement.
The CPU path states the same computation with a differentiable gather so that gloo tests cover the layout, the masks
and the gradient return.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch
import torch.distributed as dist

from halo_b200.ops import _lib
from halo_b200.ops import attention as attn_ops

TILE = 128
MAX_PIECES = 16
MAX_RANKS = 8


@dataclass
class CPLayout:
    cp_rank: int
    cp_size: int
    total: int
    cu: np.ndarray                 # the whole row's document offsets
    bounds: np.ndarray             # [P + 1] global row boundaries of the pieces
    owner: np.ndarray              # [P] rank that owns each piece
    loc: np.ndarray                # [P] first row of the piece in its owner's local order
    rows_of_rank: list             # tokens every rank holds
    written: list = field(default_factory=list)   # per rank: [(global lo, global hi, staging row)] foreign dK/dV rows it produces
    returns: list = field(default_factory=list)   # for this rank: (rank, my local row, n rows, that rank's staging row)
    stage_of: list = field(default_factory=list)  # per rank: [P] staging row of each foreign piece's first row (-1: nothing produced)

    @property
    def n_pieces(self) -> int:
        return len(self.owner)

    @property
    def local(self) -> int:
        return int(self.rows_of_rank[self.cp_rank])

    def pieces_of(self, rank: int) -> list[int]:
        return [p for p in range(self.n_pieces) if self.owner[p] == rank]

    def local_index(self, rank: int | None = None) -> np.ndarray:
        """Global token indices in ``rank``'s local order."""
        rank = self.cp_rank if rank is None else rank
        parts = [np.arange(self.bounds[p], self.bounds[p + 1]) for p in self.pieces_of(rank)]
        return np.concatenate(parts) if parts else np.zeros(0, np.int64)

    def piece_of(self, row: int) -> int:
        return int(np.searchsorted(self.bounds, row, side="right")) - 1

    def to_local(self, row: int) -> tuple[int, int]:
        """(owner rank, local row) of a global row."""
        p = self.piece_of(row)
        return int(self.owner[p]), int(row - self.bounds[p] + self.loc[p])

    def device_map(self) -> np.ndarray:
        """The table the kernels take: n_pieces, my rank, bounds[17], owner[16], loc[16], stage[16] (int32). ``stage[p]`` is the
        staging row of foreign piece ``p``'s first row (-1: the piece is mine or nothing of it is produced here)."""
        if self.n_pieces > MAX_PIECES or self.cp_size > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} context-parallel ranks ({MAX_PIECES} pieces) are supported")
        m = np.zeros(2 + 17 + 16 * 3, dtype=np.int32)
        m[0], m[1] = self.n_pieces, self.cp_rank
        m[2:2 + self.n_pieces + 1] = self.bounds
        m[2 + self.n_pieces + 1:19] = self.bounds[-1]
        m[19:19 + self.n_pieces] = self.owner
        m[35:35 + self.n_pieces] = self.loc
        stage = np.full(16, -1, dtype=np.int32)
        stage[:self.n_pieces] = self.stage_of[self.cp_rank]
        m[51:67] = stage
        return m


def _snap(cu: np.ndarray, b: int, tile: int) -> int:
    """Move a boundary that falls inside a document to the nearest multiple of ``tile`` from the document's start (or to
    the document's end when that is nearer than the next multiple)."""
    total = int(cu[-1])
    if b <= 0 or b >= total:
        return min(max(b, 0), total)
    d = int(np.searchsorted(cu, b, side="right")) - 1
    s, e = int(cu[d]), int(cu[d + 1])
    cand = s + int(round((b - s) / tile)) * tile
    return min(cand, e)


def make_layout(cu_seqlens, cp_rank: int, cp_size: int, balance: bool = True, tile: int = TILE) -> CPLayout:
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    total = int(cu[-1])
    n_pieces = 2 * cp_size if (balance and cp_size > 1) else cp_size
    bounds = [0]
    for i in range(1, n_pieces):
        bounds.append(max(bounds[-1], _snap(cu, (total * i) // n_pieces, tile)))
    bounds.append(total)
    bounds = np.asarray(bounds, dtype=np.int64)
    owner = np.asarray([p if p < cp_size else 2 * cp_size - 1 - p for p in range(n_pieces)], dtype=np.int64)
    loc = np.zeros(n_pieces, dtype=np.int64)
    rows = [0] * cp_size
    for p in range(n_pieces):                         # a rank's pieces in increasing global order
        loc[p] = rows[owner[p]]
        rows[owner[p]] += int(bounds[p + 1] - bounds[p])
    if min(rows) == 0:
        raise ValueError(f"a packed row of {total} tokens in documents of {np.diff(cu).tolist()[:8]} tokens leaves a rank "
                         f"without tokens when cut over {cp_size} ranks in {tile}-token tiles: pack longer rows")
    lay = CPLayout(cp_rank, cp_size, total, cu, bounds, owner, loc, rows)
    # what every rank produces for foreign keys: per document, the key rows below the end of the tile that holds the
    # rank's last query of that document and that lie in another rank's piece. A foreign piece's staging region starts at
    # the piece's first row and runs to its last produced row, so one offset per piece addresses it.
    lay.written, lay.stage_of = [], []
    for r in range(cp_size):
        out, srow = [], 0
        stage = np.full(n_pieces, -1, dtype=np.int64)
        mine = lay.pieces_of(r)
        for p in range(n_pieces):
            if owner[p] == r:
                continue
            plo, phi = int(bounds[p]), int(bounds[p + 1])
            runs = []
            d = max(int(np.searchsorted(cu, plo, side="right")) - 1, 0)
            while d < len(cu) - 1 and int(cu[d]) < phi:
                s, e = int(cu[d]), int(cu[d + 1])
                my_max = max((min(int(bounds[q + 1]), e) - 1 for q in mine if max(int(bounds[q]), s) < min(int(bounds[q + 1]), e)),
                             default=-1)
                if my_max >= 0:
                    tile_end = s + ((my_max - s) // tile + 1) * tile
                    lo, hi = max(s, plo), min(e, phi, tile_end)
                    if lo < hi:
                        runs.append((lo, hi))
                d += 1
            if runs:
                stage[p] = srow
                out += [(lo, hi, srow + lo - plo) for lo, hi in runs]
                srow += runs[-1][1] - plo
        lay.written.append(out)
        lay.stage_of.append(stage)
    me_pieces = set(lay.pieces_of(cp_rank))
    for r in range(cp_size):
        if r == cp_rank:
            continue
        for lo, hi, srow in lay.written[r]:
            p = lay.piece_of(lo)
            if p in me_pieces:
                lay.returns.append((r, int(lo - bounds[p] + loc[p]), hi - lo, srow))
    return lay


def staging_rows_needed(lay: CPLayout, rank: int | None = None) -> int:
    rank = lay.cp_rank if rank is None else rank
    return max((srow + hi - lo for lo, hi, srow in lay.written[rank]), default=0)


# ---- work lists in the row's global coordinates ------------------------------------------------------------------------
def build_cp_plan(layout: CPLayout, device) -> attn_ops.AttentionPlan:
    """Tile lists for the context-parallel kernels. ``fwd`` / ``bwd_q``: ``{q0, document start, 64-key sub-tiles up to the
    tile's last visible key, document end}`` for the query tiles this rank owns. ``bwd_kv`` ([n, 8]): ``{k0, first query of
    segment 1, its 64-query sub-tiles, document end, first query of segment 2, its sub-tiles, 0, 0}`` for every key tile
    (whoever owns it) that a local query can see; a segment is the part of one local piece inside the document at or
    after the key tile."""
    cu = layout.cu
    plan = attn_ops.AttentionPlan(cu_seqlens=cu, total=layout.total)
    lens = np.diff(cu)
    plan.max_seqlen = int(lens.max()) if len(lens) else 0
    device = torch.device(device) if device is not None else None
    mine = [(int(layout.bounds[p]), int(layout.bounds[p + 1])) for p in layout.pieces_of(layout.cp_rank)]
    mine = [(a, b) for a, b in mine if a < b]
    bq, bkv = [], []
    for s, e in zip(cu[:-1], cu[1:]):
        s, e = int(s), int(e)
        if e == s:
            continue
        segs = [(max(a, s), min(b, e)) for a, b in mine if max(a, s) < min(b, e)]
        if not segs:
            continue
        if len(segs) > 2:
            raise ValueError("a rank owns more than two pieces of one document")
        for a, b in segs:
            for q0 in range(s + (a - s) // TILE * TILE, b, TILE):
                last = min(q0 + TILE, e)
                bq.append((q0, s, (last - s + 63) // 64, e))
        my_max = segs[-1][1] - 1
        for k0 in range(s, my_max + 1, TILE):
            parts = []
            for a, b in segs:
                qb = max(k0, a)
                if qb < b:
                    parts.append((qb, (min(b, e) - qb + 63) // 64))
            if not parts:
                continue
            (q1, n1), (q2, n2) = parts[0], (parts[1] if len(parts) > 1 else (0, 0))
            bkv.append((k0, q1, n1, e, q2, n2, 0, 0))
    plan.cp_items = (bq, bkv)
    if device is None or device.type != "cuda":
        return plan

    def to_dev(rows, width, key):
        if not rows:
            return torch.zeros((0, width), dtype=torch.int32, device=device)
        arr = np.asarray(rows, dtype=np.int32)
        arr = arr[np.argsort(-key(arr), kind="stable")]           # longest first
        return torch.from_numpy(arr).to(device, non_blocking=True)

    plan.bwd_q = to_dev(bq, 4, lambda a: a[:, 2])
    plan.fwd = plan.bwd_q
    plan.bwd_kv = to_dev(bkv, 8, lambda a: a[:, 2] + a[:, 5])
    return plan


def covered_pairs(layout: CPLayout, plan) -> tuple[np.ndarray, np.ndarray]:
    """For tests: the (query, key) pairs the query-tile list and the key-tile list of ``plan`` visit, as boolean
    ``[total, total]`` matrices (causal and document masks applied as the kernels apply them)."""
    T = layout.total
    bq, bkv = plan.cp_items
    fwd = np.zeros((T, T), bool)
    for q0, s, n64, e in bq:
        for q in range(q0, min(q0 + TILE, e)):
            hi = min(s + 64 * n64, e)
            fwd[q, s:min(q + 1, hi)] = True
    kv = np.zeros((T, T), bool)
    for k0, q1, n1, e, q2, n2, _, _ in bkv:
        for qb, n in ((q1, n1), (q2, n2)):
            for q in range(qb, min(qb + 64 * n, e)):
                for k in range(k0, min(k0 + TILE, e)):
                    if k <= q:
                        assert not kv[q, k], "a (query, key) pair is visited twice"
                        kv[q, k] = True
    return fwd, kv


# ---- differentiable gather for the PyTorch path ---------------------------------------------------------------------------
class _GatherRows(torch.autograd.Function):
    """Every rank's local rows assembled into the whole row ``[total, C]`` (ranks may hold different counts); backward:
    the sum over ranks of the gradient, cut back to the local rows."""

    @staticmethod
    def forward(ctx, x, layout: CPLayout, group):
        world = dist.get_world_size(group)
        most = max(layout.rows_of_rank)
        padded = x.new_zeros((most, x.shape[1]))
        padded[:x.shape[0]] = x
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded, group=group)
        out = x.new_zeros((layout.total, x.shape[1]))
        for r in range(world):
            idx = torch.from_numpy(layout.local_index(r))
            out[idx] = parts[r][:len(idx)]
        ctx.group, ctx.layout = group, layout
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        idx = torch.from_numpy(ctx.layout.local_index())
        return g[idx], None, None


class CPExchange:
    """Symmetric buffers and barriers of one context-parallel group (GPU path).

    ``kv``: this rank's published keys | values in local order (peers read it). ``dkv``: dK | dV this rank produced for
    key rows, read by their owners. ``mirror`` (plain local memory, indexed by GLOBAL row): the keys | values this rank's
    kernels read - its own rows and the foreign rows it needs, fetched once per exchange. With ``direct_reads`` the
    kernels skip the mirror and read every foreign tile from its owner over NVLink: fine when few foreign rows are
    touched, but every CTA's read of a tile crosses the link again (one 64k-token document on two GPUs moves 137 GB per
    layer that way and runs five times slower than the mirror), so it is an option, not the default."""

    def __init__(self, group, device, max_local_rows: int, max_row_tokens: int, kv_cols: int, direct_reads: bool | None = None):
        import torch.distributed._symmetric_memory as symm

        from halo_b200 import env

        self.group, self.device = group, torch.device(device)
        self.n_ranks, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.direct_reads = env.cp_direct_reads() if direct_reads is None else bool(direct_reads)
        self.kv = symm.empty((max_local_rows, kv_cols), dtype=torch.bfloat16, device=self.device)
        self.dkv = symm.empty((max(max_row_tokens, 8), kv_cols), dtype=torch.bfloat16, device=self.device)
        # rows a tile reads past a document's end are masked, but must hold finite values
        self.kv.zero_()
        self.dkv.zero_()
        self.mirror = torch.zeros((max(max_row_tokens, 8), kv_cols), dtype=torch.bfloat16, device=self.device)
        self.mirror_version = 0
        self.h_kv = symm.rendezvous(self.kv, group)
        self.h_dkv = symm.rendezvous(self.dkv, group)
        self.kv_ptrs = list(self.h_kv.buffer_ptrs)
        self.dkv_ptrs = list(self.h_dkv.buffer_ptrs)
        self.kv_ptr_array = (_lib.c_void_p * self.n_ranks)(*self.kv_ptrs)
        self.mirror_ptr_array = (_lib.c_void_p * 1)(self.mirror.data_ptr())
        self.row_bytes = kv_cols * 2
        self.max_local_rows, self.max_row_tokens = max_local_rows, max(max_row_tokens, 8)

    def barrier(self) -> None:
        self.h_kv.barrier(channel=3)

    def publish(self, k: torch.Tensor, v: torch.Tensor) -> None:
        n, kvd = k.shape
        if n > self.max_local_rows:
            raise ValueError(f"{n} local rows exceed the exchange buffer's {self.max_local_rows}")
        self.kv[:n, :kvd].copy_(k)
        self.kv[:n, kvd:].copy_(v)

    def pull(self, dst: torch.Tensor, base_ptr: int, first_row: int, n_rows: int, accumulate: bool) -> None:
        rc = _lib.lib().halo_peer_pull(_lib.ptr(dst), _lib.c_void_p(base_ptr + first_row * self.row_bytes),
                                       _lib.c_ll(n_rows * self.row_bytes), _lib.c_int(1 if accumulate else 0),
                                       _lib.stream_ptr(self.device))
        _lib.check(rc, "halo_peer_pull")

    def fetch_mirror(self, k: torch.Tensor, v: torch.Tensor, layout: CPLayout) -> int:
        """COLLECTIVE: publish this rank's rows, then fill the mirror with them and with the foreign rows this rank's
        queries can see (each crosses NVLink once). Returns the mirror's version."""
        if layout.total > self.max_row_tokens:
            raise ValueError(f"a row of {layout.total} tokens exceeds the exchange's {self.max_row_tokens}")
        kvd = k.shape[1]
        self.publish(k, v)
        self.barrier()                          # every rank's rows are in place
        for p in layout.pieces_of(layout.cp_rank):
            lo, hi, at = int(layout.bounds[p]), int(layout.bounds[p + 1]), int(layout.loc[p])
            if hi > lo:
                self.mirror[lo:hi, :kvd].copy_(k[at:at + hi - lo])
                self.mirror[lo:hi, kvd:].copy_(v[at:at + hi - lo])
        for lo, hi, _ in layout.written[layout.cp_rank]:
            rank, row = layout.to_local(lo)
            self.pull(self.mirror[lo:hi], self.kv_ptrs[rank], row, hi - lo, accumulate=False)
        self.barrier()                          # peers are done reading before anybody publishes again
        self.mirror_version += 1
        return self.mirror_version


def _map_array(layout: CPLayout):
    m = layout.device_map()
    return (_lib.c_int * len(m))(*[int(x) for x in m])


def _mirror_map(total: int):
    """Key table of the mirror: one piece covering the row, owned by nobody, staged at its global rows."""
    m = np.zeros(2 + 17 + 16 * 3, dtype=np.int32)
    m[0], m[1] = 1, -1
    m[3:19] = total
    m[51:67] = -1
    m[51] = 0
    return (_lib.c_int * len(m))(*[int(x) for x in m])


class _CPFlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, layout: CPLayout, plan, exchange: CPExchange, n_heads, n_kv_heads, scale):
        Tl = layout.local
        dev = q.device
        D = attn_ops.HEAD_DIM
        kvd = n_kv_heads * D
        version = 0
        if exchange.direct_reads:
            if staging_rows_needed(layout) > exchange.max_row_tokens:
                raise ValueError("the key/value gradient staging buffer is too small for this row")
            exchange.publish(k, v)
            exchange.barrier()                      # every rank's keys and values are in place
            ptrs, n_bufs, rows, kv_map = exchange.kv_ptr_array, exchange.n_ranks, exchange.max_local_rows, _map_array(layout)
        else:
            version = exchange.fetch_mirror(k, v, layout)
            ptrs, n_bufs, rows, kv_map = exchange.mirror_ptr_array, 1, exchange.max_row_tokens, _mirror_map(layout.total)
        o = torch.empty((Tl, n_heads * D), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((n_heads, Tl), dtype=torch.float32, device=dev)
        L = _lib.lib()
        rc = L.halo_attn_cp_fwd(
            _lib.ptr(q), ptrs, _lib.c_int(n_bufs), _lib.c_ll(rows),
            _lib.c_ll(2 * kvd), _lib.c_int(kvd), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(plan.fwd), _lib.c_int(plan.fwd.shape[0]),
            _lib.c_ll(Tl), _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(D), _lib.c_ll(attn_ops._ld(q)),
            _lib.c_ll(attn_ops._ld(o)), _lib.c_float(scale), _map_array(layout), kv_map, _lib.ptr(_lib.status_word(dev)),
            _lib.stream_ptr(dev))
        _lib.check(rc, "halo_attn_cp_fwd")
        if exchange.direct_reads:
            exchange.barrier()                      # peers are done reading before the next layer publishes
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.meta = (layout, plan, exchange, n_heads, n_kv_heads, scale, version)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        layout, plan, exchange, n_heads, n_kv_heads, scale, version = ctx.meta
        Tl = layout.local
        dev = do.device
        D = attn_ops.HEAD_DIM
        kvd = n_kv_heads * D
        do = do.contiguous()
        if exchange.direct_reads:
            exchange.publish(k, v)
            exchange.barrier()
            ptrs, n_bufs, rows, kv_map = exchange.kv_ptr_array, exchange.n_ranks, exchange.max_local_rows, _map_array(layout)
        else:
            # the mirror still holds this layer's rows when its forward was the last exchange (per-layer recomputation
            # runs a layer's forward right before its backward); every rank sees the same sequence, so all agree
            if exchange.mirror_version != version:
                exchange.fetch_mirror(k, v, layout)
            ptrs, n_bufs, rows, kv_map = exchange.mirror_ptr_array, 1, exchange.max_row_tokens, _mirror_map(layout.total)
        dq = torch.empty_like(q)
        dkv = torch.zeros((Tl, 2 * kvd), dtype=torch.bfloat16, device=dev)
        delta = torch.empty((n_heads, Tl), dtype=torch.float32, device=dev)
        dk, dv = dkv[:, :kvd], dkv[:, kvd:]
        stage_k, stage_v = exchange.dkv[:, :kvd], exchange.dkv[:, kvd:]
        L = _lib.lib()
        ld = attn_ops._ld
        rc = L.halo_attn_cp_bwd(
            _lib.ptr(q), ptrs, _lib.c_int(n_bufs), _lib.c_ll(rows),
            _lib.c_ll(2 * kvd), _lib.c_int(kvd), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(delta), _lib.ptr(dq),
            _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(stage_k), _lib.ptr(stage_v), _lib.c_ll(2 * kvd),
            _lib.ptr(plan.bwd_kv), _lib.c_int(plan.bwd_kv.shape[0]), _lib.ptr(plan.bwd_q), _lib.c_int(plan.bwd_q.shape[0]),
            _lib.c_ll(Tl), _lib.c_int(n_heads), _lib.c_int(n_kv_heads), _lib.c_int(D), _lib.c_ll(ld(q)), _lib.c_ll(ld(o)),
            _lib.c_ll(ld(do)), _lib.c_ll(ld(dq)), _lib.c_ll(ld(dk)), _lib.c_ll(ld(dv)), _lib.c_float(scale), _map_array(layout),
            kv_map, _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev))
        _lib.check(rc, "halo_attn_cp_bwd")
        exchange.barrier()                      # every rank's dK / dV are complete
        if exchange.direct_reads:
            for rank, my_row, n, src_row in layout.returns:          # ascending rank: a fixed summation order
                exchange.pull(dkv[my_row:my_row + n], exchange.dkv_ptrs[rank], src_row, n, accumulate=True)
        else:
            # own contribution first (every local key tile was visited by a local query), then the peers' in rank order
            for p in layout.pieces_of(layout.cp_rank):
                lo, hi, at = int(layout.bounds[p]), int(layout.bounds[p + 1]), int(layout.loc[p])
                if hi > lo:
                    dkv[at:at + hi - lo].copy_(exchange.dkv[lo:hi])
            for rank in range(layout.cp_size):
                if rank == layout.cp_rank:
                    continue
                for lo, hi, _ in layout.written[rank]:
                    owner, row = layout.to_local(lo)
                    if owner == layout.cp_rank:
                        exchange.pull(dkv[row:row + hi - lo], exchange.dkv_ptrs[rank], lo, hi - lo, accumulate=True)
        exchange.barrier()
        return dq, dkv[:, :kvd], dkv[:, kvd:], None, None, None, None, None, None


def cp_attention(q, k, v, layout: CPLayout, plan, group, exchange: CPExchange | None, n_heads: int, n_kv_heads: int,
                 scale: float | None = None):
    """Causal attention of this rank's tokens of a packed row. q: [T_local, Hq*D]; k, v: [T_local, Hkv*D]."""
    D = q.shape[1] // n_heads
    scale = float(scale if scale is not None else D**-0.5)
    if q.is_cuda:
        if exchange is None:
            raise RuntimeError("the GPU context-parallel path needs a CPExchange (symmetric K/V buffers)")
        return _CPFlashAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), layout, plan, exchange, n_heads,
                                       n_kv_heads, scale)
    # PyTorch path: assemble the whole row's K/V (differentiably), attend with the local queries scattered into an
    # otherwise zero query tensor, keep the local rows
    k_all, v_all = _GatherRows.apply(k, layout, group), _GatherRows.apply(v, layout, group)
    idx = torch.from_numpy(layout.local_index())
    q_all = q.new_zeros((layout.total, q.shape[1])).index_put((idx,), q)
    o_all = attn_ops.attention_reference(q_all, k_all, v_all, layout.cu, n_heads, n_kv_heads, scale)
    return o_all[idx]


class ContextParallel:
    """Per-run state the model's forward context carries when ``context_parallel_size > 1``."""

    def __init__(self, group, device, cfg, max_row_tokens: int, balance: bool = True):
        self.group = group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = torch.device(device)
        self.balance = balance
        self.exchange = None
        if self.device.type == "cuda":
            # a boundary moves by at most half a tile; a rank's pieces have four boundaries
            local = max_row_tokens // self.size + 4 * TILE
            self.exchange = CPExchange(group, device, local, max_row_tokens + TILE, 2 * cfg.num_key_value_heads * cfg.head_dim)

    def layout_of(self, cu_seqlens) -> CPLayout:
        return make_layout(cu_seqlens, self.rank, self.size, self.balance)

    def layout_and_plan(self, cu_seqlens):
        lay = self.layout_of(cu_seqlens)
        return lay, build_cp_plan(lay, self.device)


def slice_batch(batch, cp_rank: int, cp_size: int, balance: bool = True):
    """This rank's tokens of a packed batch; ``cu_seqlens`` stays the whole row's (the layout needs it)."""
    from halo_b200.data.packing import PackedBatch

    lay = make_layout(batch.cu_seqlens, cp_rank, cp_size, balance)
    idx = torch.from_numpy(lay.local_index())
    labels = batch.labels[idx]
    return PackedBatch(batch.input_ids[idx], batch.position_ids[idx], labels, batch.cu_seqlens, int((labels != -100).sum()))


def chunk_bounds(total: int, n: int, rank: int) -> tuple[int, int]:
    """Equal contiguous cut of ``total`` tokens (the tensor-parallel token shards)."""
    if total % n:
        raise ValueError(f"a packed row of {total} tokens cannot be cut into {n} equal chunks: pad the row")
    c = total // n
    return rank * c, (rank + 1) * c
