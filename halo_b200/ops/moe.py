"""Routed-expert FFN: router top-k, dispatch to the expert-owning rank, grouped SwiGLU FFN on
the tcgen05 grouped GEMM, weighted combine; forward and backward, as one autograd node.

Data flow for one layer on a rank that owns ``E_local`` of ``E`` experts (``N`` ranks):

  counts    histogram of this rank's [T, k] routing over all E experts        (route_count)
  exchange  all ranks' histograms -> every rank derives every rank's receive layout (transport)
  place     each (token, k) slot gets its row in the owner's receive buffer   (route_place)
  dispatch  token rows are pushed into the owners' buffers (peer stores)      (dispatch_rows)
  FFN       gate_up GEMM with SwiGLU epilogue, down GEMM, per-expert tile lists built on device
  combine   each token pulls its k expert rows back (peer loads), weights and sums them in fp32

Backward runs the same movement in reverse: dout rows are pushed to the experts together with the
routing weights, the expert side forms dy and the routing-weight gradient, the grouped GEMMs
produce the weight and input gradients, and the input-gradient rows are pulled back and summed.
No host synchronisation happens anywhere: segment sizes stay on the device and size the GEMM tile
lists there; buffers are provisioned from a capacity bound that is checked on the device.

Replaces DeepEP dispatch/combine, the Triton route sort / permute kernels and ``F.grouped_mm``
(halo/distributed/expert_parallel/moe_layer/layer.py:301-342,
halo/distributed/expert_parallel/moe_layer/compute.py:222-242, 357-361).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import _lib
from .gemm import EPI_STORE_BF16, EPI_SWIGLU


# ---------------------------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------------------------
def router_topk_reference(logits: torch.Tensor, k: int, renorm: bool, sel_bias: torch.Tensor | None = None):
    probs = torch.softmax(logits.float(), dim=-1)
    if sel_bias is None:
        w, idx = torch.topk(probs, k, dim=-1)
    else:
        # the balancing bias ranks experts; the weights stay the unbiased probabilities
        _, idx = torch.topk(probs + sel_bias.float(), k, dim=-1)
        w = probs.gather(-1, idx)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return idx.to(torch.int32), w


def router_grouped_topk(logits: torch.Tensor, k: int, renorm: bool, sel_bias: torch.Tensor | None = None, n_group: int = 1,
                        topk_group: int = 1, scaling: float = 1.0, score: str = "sigmoid", eps: float = 1e-20):
    """Group-limited routing (DeepSeek-V3 / GLM-4 with sigmoid scores, Mistral 4 with softmax scores): the ranking adds
    the selection bias and, with ``n_group > 1``, keeps only the ``topk_group`` groups of experts whose two best biased
    scores sum highest; the weights are the unbiased scores of the chosen experts, renormalised and scaled. Tensor
    ops with autograd (the score matrix is ``[T, E]``: small beside the expert products)."""
    scores = torch.sigmoid(logits.float()) if score == "sigmoid" else torch.softmax(logits.float(), dim=-1)
    choice = scores if sel_bias is None else scores + sel_bias.float()
    if n_group > 1:
        T, E = choice.shape
        grouped = choice.view(T, n_group, E // n_group)
        group_scores = grouped.topk(min(2, E // n_group), dim=-1).values.sum(-1)
        keep = torch.zeros_like(group_scores, dtype=torch.bool).scatter_(1, group_scores.topk(topk_group, dim=-1).indices, True)
        choice = choice.masked_fill(~keep[:, :, None].expand_as(grouped).reshape(T, E), 0.0)
    idx = choice.detach().topk(k, dim=-1).indices
    w = scores.gather(-1, idx)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + eps)
    return idx.to(torch.int32), w * scaling


def router_sigmoid_topk(logits, k, renorm, sel_bias=None, n_group=1, topk_group=1, scaling=1.0):
    return router_grouped_topk(logits, k, renorm, sel_bias, n_group, topk_group, scaling, "sigmoid")


class _RouterTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, renorm, sel_bias=None):
        T, E = logits.shape
        idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
        rc = _lib.lib().halo_router_topk_fwd(
            _lib.ptr(logits), _lib.ptr(idx), _lib.ptr(w), _lib.c_void_p(0), _lib.ptr(sel_bias), _lib.c_ll(T),
            _lib.c_int(E), _lib.c_int(k), _lib.c_int(1 if renorm else 0), _lib.stream_ptr(logits.device),
        )
        _lib.check(rc, "halo_router_topk_fwd")
        ctx.save_for_backward(logits, idx)
        ctx.meta = (k, renorm)
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _gidx, gw):
        logits, idx = ctx.saved_tensors
        k, renorm = ctx.meta
        T, E = logits.shape
        dl = torch.empty_like(logits)
        rc = _lib.lib().halo_router_topk_bwd(
            _lib.ptr(logits), _lib.ptr(idx), _lib.ptr(gw.contiguous().float()), _lib.ptr(dl), _lib.c_ll(T),
            _lib.c_int(E), _lib.c_int(k), _lib.c_int(1 if renorm else 0), _lib.stream_ptr(logits.device),
        )
        _lib.check(rc, "halo_router_topk_bwd")
        return dl, None, None, None


def router_topk(logits: torch.Tensor, k: int, renorm: bool = True, sel_bias: torch.Tensor | None = None):
    """softmax over experts, top-k, optional renormalisation. logits: fp32 [T, E]. ``sel_bias`` ([E],
    no gradient) is added to the probabilities for the ranking only (auxiliary-loss-free balancing).
    Returns ``(idx int32 [T, k], weights fp32 [T, k])``."""
    E = logits.shape[-1]
    if not logits.is_cuda or E % 32 or E > 256 or k > 16:
        return router_topk_reference(logits, k, renorm, sel_bias)
    if sel_bias is not None:
        sel_bias = sel_bias.detach().float().contiguous()
    return _RouterTopK.apply(logits.float().contiguous(), k, renorm, sel_bias)


# ---------------------------------------------------------------------------------------------
# transport: who owns which buffer and how ranks agree on counts
# ---------------------------------------------------------------------------------------------
class LocalTransport:
    """Single-rank transport: every expert is local, buffers are ordinary device tensors."""

    n_ranks = 1
    rank = 0

    def __init__(self, capacity_factor: float = 1.0):
        from halo_b200 import env

        self.capacity_factor = capacity_factor
        self.fused = env.moe_fused()
        self.seq = 0
        self.max_tiles = 0
        self.n_experts = 0
        self._ctrl = None
        self._live: dict[int, torch.Tensor] = {}

    def capacity(self, n_slots: int, n_local_experts: int) -> int:
        # every slot lands here; each expert segment is padded to a multiple of 128 rows
        return n_slots + 128 * n_local_experts

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        return counts.reshape(1, -1)

    def buffer(self, name: str, rows: int, cols: int, dtype: torch.dtype, device) -> torch.Tensor:
        return torch.empty((rows, cols), dtype=dtype, device=device)

    def peer_table(self, buf: torch.Tensor):
        """Host array of every rank's base pointer for this buffer (here: just ours); it travels to
        the kernels by value."""
        return (_lib.c_void_p * 1)(buf.data_ptr())

    # ---- control block of the fused path (one rank: the handshake is with itself) ----
    def prepare_ctrl(self, n_experts: int, capacity: int, device) -> None:
        max_tiles = capacity // 128
        if self._ctrl is None or self.n_experts != n_experts or self.max_tiles < max_tiles or self._ctrl.device != device:
            self.n_experts, self.max_tiles = n_experts, max_tiles
            self._ctrl = torch.zeros(2 * n_experts + 1 + 2 * max_tiles, dtype=torch.int32, device=device)
            self.seq = 0

    def next_seq(self) -> int:
        self.seq += 1
        return self.seq

    def ctrl_table(self):
        return (_lib.c_void_p * 1)(self._ctrl.data_ptr())

    def arrive_table(self, seq: int):
        off = 4 * (2 * self.n_experts + 1 + (seq & 1) * self.max_tiles)
        return (_lib.c_void_p * 1)(self._ctrl.data_ptr() + off)

    def barrier(self, channel: int = 0) -> None:
        """All ranks' writes issued before this point are visible to reads issued after it."""

    def barrier_before_push(self) -> None:
        """Peers are done reading the buffers this rank is about to fill (nothing to do on one rank)."""

    def side_stream(self, device):
        return None

    @property
    def transient_buffers(self) -> bool:
        return False


@dataclass
class RoutingState:
    """Everything derived from one layer's routing; kept for the backward."""

    n_tokens: int
    top_k: int
    n_experts: int
    n_local: int
    capacity: int
    topk_idx: torch.Tensor          # int32 [T, k]
    slot_row: torch.Tensor          # int32 [T*k]
    seg_start: torch.Tensor         # int32 [E_local]
    seg_rows: torch.Tensor          # int32 [E_local]
    total_rows: torch.Tensor        # int32 [1]
    counts: torch.Tensor            # int32 [E] this rank's slots per expert
    lists: dict = field(default_factory=dict)
    # fused path only
    send_slot: torch.Tensor | None = None    # int32 [T*k] slot ids in destination order
    units: torch.Tensor | None = None        # push units (bytes)
    n_units: torch.Tensor | None = None      # int32 [1]
    tiles: torch.Tensor | None = None        # receive-buffer tiles in arrival order (bytes)
    n_tiles: torch.Tensor | None = None      # int32 [1]
    seq: int = 0                             # control-block call number of the forward


def _work_bytes() -> int:
    return int(_lib.lib().halo_gemm_work_bytes())


def plan_routing(topk_idx: torch.Tensor, n_experts: int, transport) -> RoutingState:
    T, k = topk_idx.shape
    capacity = transport.capacity(T * k, n_experts // transport.n_ranks)
    dev = topk_idx.device
    L = _lib.lib()
    n_slots = T * k
    idx = topk_idx.contiguous()
    n_blocks = L.halo_route_blocks(_lib.c_ll(n_slots))
    block_hist = torch.empty((max(n_blocks, 1), n_experts), dtype=torch.int32, device=dev)
    counts = torch.empty(n_experts, dtype=torch.int32, device=dev)
    s = _lib.stream_ptr(dev)
    _lib.check(L.halo_route_count(_lib.ptr(idx), _lib.c_ll(n_slots), _lib.c_int(n_experts), _lib.ptr(block_hist),
                                  _lib.ptr(counts), s), "halo_route_count")
    counts_all = transport.exchange_counts(counts).contiguous()
    n_local = n_experts // transport.n_ranks
    seg_start = torch.empty(n_local, dtype=torch.int32, device=dev)
    seg_rows = torch.empty(n_local, dtype=torch.int32, device=dev)
    dst_base = torch.empty(n_experts, dtype=torch.int32, device=dev)
    total_rows = torch.empty(1, dtype=torch.int32, device=dev)
    _lib.check(L.halo_route_layout(_lib.ptr(counts_all), _lib.c_int(transport.n_ranks), _lib.c_int(n_experts),
                                   _lib.c_int(transport.rank), _lib.ptr(seg_start), _lib.ptr(seg_rows),
                                   _lib.ptr(dst_base), _lib.ptr(total_rows), _lib.c_int(capacity),
                                   _lib.ptr(_lib.status_word(dev)), s), "halo_route_layout")
    slot_row = torch.empty(n_slots, dtype=torch.int32, device=dev)
    _lib.check(L.halo_route_place(_lib.ptr(idx), _lib.c_ll(n_slots), _lib.c_int(n_experts), _lib.ptr(block_hist),
                                  _lib.ptr(dst_base), _lib.ptr(slot_row), s), "halo_route_place")
    return RoutingState(
        n_tokens=T, top_k=k, n_experts=n_experts, n_local=n_local,
        capacity=capacity, topk_idx=idx, slot_row=slot_row,
        seg_start=seg_start, seg_rows=seg_rows, total_rows=total_rows, counts=counts,
    )


def _alloc(transport, shape, dtype, dev):
    """A temporary for an expert op. A lane of a multi-lane transport runs on its own stream; PyTorch's caching
    allocator keeps one pool per stream, and with several GB of temporaries per lane those pools cannot lend to
    each other, so an almost full device would spend its time releasing and re-mapping segments. Lanes therefore
    take their temporaries from the pool of the stream that issued the op and mark them as used by the lane's
    stream (the block is not handed out again before the lane's work on it has finished)."""
    home = getattr(transport, "alloc_stream", None)
    if home is None:
        return torch.empty(shape, dtype=dtype, device=dev)
    with torch.cuda.stream(home):
        t = torch.empty(shape, dtype=dtype, device=dev)
    t.record_stream(transport.stream)
    side = getattr(transport, "_side", None)
    if side is not None:
        t.record_stream(side)
    return t


_PAIR_ENABLED = None


def _pair_ok(k_dim: int, swiglu: bool) -> int:
    """Which GEMM kernel runs a grouped product. On the 30B-A3B expert shapes the CTA-pair form (256-row tiles)
    shortens the kernels themselves by only 1-5 % and the step as a whole measured no faster, so grouped products
    stay on the single-CTA kernel unless HALO_GEMM_PAIR=2 forces the pair form everywhere."""
    global _PAIR_ENABLED
    if _PAIR_ENABLED is None:
        _PAIR_ENABLED = int(_lib.lib().halo_gemm_pair_enabled())
    return int(_PAIR_ENABLED == 2 and not swiglu)


def _tile_list(state: RoutingState, kind: str, pair: int = 0, **kw):
    """Device tile list for one grouped product shape, cached per routing state."""
    key = (kind, pair, tuple(sorted(kw.items())))
    hit = state.lists.get(key)
    if hit is not None:
        return hit
    L = _lib.lib()
    dev = state.slot_row.device
    wb = _work_bytes()
    s = _lib.stream_ptr(dev)
    count = torch.empty(1, dtype=torch.int32, device=dev)
    if kind == "m":
        tile_n = 128 if kw["swiglu_f"] else 256
        width = kw["swiglu_f"] if kw["swiglu_f"] else kw["n_cols"]
        tiles_n = (width + tile_n - 1) // tile_n
        max_items = (state.capacity // 128 + state.n_local) * tiles_n
        lst = torch.empty(max_items * wb, dtype=torch.uint8, device=dev)
        _lib.check(L.halo_plan_grouped_m(
            _lib.ptr(state.seg_start), _lib.ptr(state.seg_rows), _lib.c_int(state.n_local), _lib.c_int(kw["n_cols"]),
            _lib.c_int(kw["k_dim"]), _lib.c_int(kw["b_mn_stride"]), _lib.c_int(kw["b_k_stride"]),
            _lib.c_int(kw["swiglu_f"]), _lib.ptr(lst), _lib.ptr(count), _lib.c_int(max_items), s, _lib.c_int(pair)),
            "halo_plan_grouped_m")
    else:
        tiles = ((kw["m_dim"] + 127) // 128) * ((kw["n_dim"] + 255) // 256)
        max_items = tiles * state.n_local
        lst = torch.empty(max_items * wb, dtype=torch.uint8, device=dev)
        _lib.check(L.halo_plan_grouped_k(
            _lib.ptr(state.seg_start), _lib.ptr(state.seg_rows), _lib.c_int(state.n_local), _lib.c_int(kw["m_dim"]),
            _lib.c_int(kw["n_dim"]), _lib.ptr(lst), _lib.ptr(count), _lib.c_int(max_items), s, _lib.c_int(pair)),
            "halo_plan_grouped_k")
    state.lists[key] = (lst, count)
    return lst, count


def _gemm_list(a, b2d, c, lst_cnt, a_mn, b_mn, epi, aux=None, swiglu_f=0, alpha=1.0, pair=0):
    lst, cnt = lst_cnt
    L = _lib.lib()
    rc = L.halo_gemm_bf16_list(
        _lib.ptr(a), _lib.c_ll(a.shape[0]), _lib.c_ll(a.shape[1]), _lib.c_ll(a.stride(0)),
        _lib.ptr(b2d), _lib.c_ll(b2d.shape[0]), _lib.c_ll(b2d.shape[1]), _lib.c_ll(b2d.stride(0)),
        _lib.ptr(c), _lib.ptr(aux), _lib.c_ll(c.stride(0)), _lib.c_ll(aux.stride(0) if aux is not None else 0),
        _lib.c_int(a_mn), _lib.c_int(b_mn), _lib.c_int(epi), _lib.c_float(alpha), _lib.c_int(swiglu_f),
        _lib.ptr(lst), _lib.ptr(cnt), _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr(a.device), _lib.c_int(pair),
    )
    _lib.check(rc, "halo_gemm_bf16_list")


def grouped_swiglu_ffn_fwd(state: RoutingState, x_rows, w_gate_up, w_down, save_pre: bool, transport=None):
    """x_rows: [cap, H] grouped by expert. Returns (y_rows [cap, H], act [cap, F], pre [cap, 2F] | None)."""
    E, F2, H = w_gate_up.shape
    F = F2 // 2
    cap = x_rows.shape[0]
    dev = x_rows.device
    act = _alloc(transport, (cap, F), torch.bfloat16, dev)
    pre = _alloc(transport, (cap, F2), torch.bfloat16, dev) if save_pre else None
    lst1 = _tile_list(state, "m", n_cols=F2, k_dim=H, b_mn_stride=F2, b_k_stride=0, swiglu_f=F)
    _gemm_list(x_rows, w_gate_up.reshape(E * F2, H), act, lst1, 0, 0, EPI_SWIGLU, aux=pre, swiglu_f=F)
    return act, pre


def grouped_biased_glu_fwd(state: RoutingState, x_rows, w_gate_up, gate_up_bias, limit: float, alpha: float, transport=None):
    """Experts with bias vectors and a clamped GLU: the first product's epilogue adds the expert's bias to the
    accumulators (the bias bank is indexed like the rows of the weight bank), stores the biased pre-activations (the
    backward reads them) and writes ``(up + 1) * gate * sigmoid(alpha gate)`` of the clamped halves.
    Returns (act [cap, F], pre [cap, 2F])."""
    E, F2, H = w_gate_up.shape
    F = F2 // 2
    cap = x_rows.shape[0]
    dev = x_rows.device
    act = _alloc(transport, (cap, F), torch.bfloat16, dev)
    pre = _alloc(transport, (cap, F2), torch.bfloat16, dev)
    lst, cnt = _tile_list(state, "m", n_cols=F2, k_dim=H, b_mn_stride=F2, b_k_stride=0, swiglu_f=F)
    b2d = w_gate_up.reshape(E * F2, H)
    _lib.check(_lib.lib().halo_gemm_bf16_list_glu(
        _lib.ptr(x_rows), _lib.c_ll(x_rows.shape[0]), _lib.c_ll(x_rows.shape[1]), _lib.c_ll(x_rows.stride(0)),
        _lib.ptr(b2d), _lib.c_ll(b2d.shape[0]), _lib.c_ll(b2d.shape[1]), _lib.c_ll(b2d.stride(0)),
        _lib.ptr(act), _lib.ptr(pre), _lib.c_ll(act.stride(0)), _lib.c_ll(pre.stride(0)), _lib.c_int(F),
        _lib.ptr(gate_up_bias), _lib.c_float(limit), _lib.c_float(alpha), _lib.ptr(lst), _lib.ptr(cnt),
        _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)), "halo_gemm_bf16_list_glu")
    return act, pre


def _expert_colsum(state: RoutingState, src, row_w, n_cols: int):
    """Per-expert column sums of a row buffer (weighted per row when ``row_w`` is given) -> fp32 [E_local, n_cols]."""
    out = torch.empty((state.n_local, n_cols), dtype=torch.float32, device=src.device)
    _lib.check(_lib.lib().halo_expert_colsum(
        _lib.ptr(src), _lib.ptr(row_w), _lib.ptr(out), _lib.ptr(state.seg_start), _lib.ptr(state.seg_rows),
        _lib.c_int(state.n_local), _lib.c_int(n_cols), _lib.c_int(state.capacity), _lib.stream_ptr(src.device)),
        "halo_expert_colsum")
    return out


def grouped_down_fwd(state: RoutingState, act, w_down, out_rows):
    E, H, F = w_down.shape
    pair = _pair_ok(F, False)
    lst2 = _tile_list(state, "m", pair, n_cols=H, k_dim=F, b_mn_stride=H, b_k_stride=0, swiglu_f=0)
    _gemm_list(act, w_down.reshape(E * H, F), out_rows, lst2, 0, 0, EPI_STORE_BF16, pair=pair)
    return out_rows


# ---------------------------------------------------------------------------------------------
# fused path: counts through peer memory, dispatch inside GEMM 1, combine inside the last GEMM's epilogue
# ---------------------------------------------------------------------------------------------
# When a list, the fused path appends (phase name, CUDA event) marks to it: the microbenchmarks read phase durations
# from consecutive marks. None (the default) records nothing.
PHASE_MARKS: list | None = None


def _mark(name: str, dev) -> None:
    if PHASE_MARKS is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(dev))
        PHASE_MARKS.append((name, ev))


def _fused(transport) -> bool:
    return bool(getattr(transport, "fused", False)) and hasattr(transport, "ctrl_table")


def plan_routing_fused(topk_idx: torch.Tensor, n_experts: int, transport) -> RoutingState:
    """Routing state of one call on the fused path: this rank's histogram, the handshake that hands it to every peer
    and derives every receive layout, slot placement with the destination-ordered send list, the push units and the
    receive-buffer tiles in arrival order. All on the device; nothing is read back."""
    T, k = topk_idx.shape
    if T * k >= 1 << 24 or n_experts > 256:
        raise ValueError(f"the fused expert path tags rows with 24-bit slot numbers and plans up to 256 experts "
                         f"(got {T * k} slots, {n_experts} experts); set HALO_MOE_FUSED=0 for larger calls")
    n_ranks, me = transport.n_ranks, transport.rank
    n_local = n_experts // n_ranks
    capacity = transport.capacity(T * k, n_local)
    dev = topk_idx.device
    if hasattr(transport, "prepare_ctrl"):
        transport.prepare_ctrl(n_experts, capacity, dev)
    L = _lib.lib()
    n_slots = T * k
    idx = topk_idx.contiguous()
    n_blocks = L.halo_route_blocks(_lib.c_ll(n_slots))
    block_hist = torch.empty((max(n_blocks, 1), n_experts), dtype=torch.int32, device=dev)
    counts = torch.empty(n_experts, dtype=torch.int32, device=dev)
    s = _lib.stream_ptr(dev)
    status = _lib.ptr(_lib.status_word(dev))
    _lib.check(L.halo_route_count(_lib.ptr(idx), _lib.c_ll(n_slots), _lib.c_int(n_experts), _lib.ptr(block_hist),
                                  _lib.ptr(counts), s), "halo_route_count")
    ints = torch.empty(2 * n_local + 2 * n_experts + 3, dtype=torch.int32, device=dev)
    seg_start, seg_rows = ints[:n_local], ints[n_local:2 * n_local]
    dst_base = ints[2 * n_local:2 * n_local + n_experts]
    my_prefix = ints[2 * n_local + n_experts:2 * n_local + 2 * n_experts]
    total_rows, n_units, n_tiles = (ints[2 * n_local + 2 * n_experts + i:2 * n_local + 2 * n_experts + i + 1] for i in range(3))
    seq = transport.next_seq()
    ctrl = transport.ctrl_table()
    _lib.check(L.halo_moe_handshake(ctrl, _lib.c_int(me), _lib.c_int(n_ranks), _lib.c_int(n_experts), _lib.c_int(seq),
                                    _lib.c_int(transport.max_tiles), _lib.ptr(counts), _lib.c_int(capacity),
                                    _lib.ptr(seg_start), _lib.ptr(seg_rows), _lib.ptr(dst_base), _lib.ptr(total_rows),
                                    _lib.ptr(my_prefix), status, s), "halo_moe_handshake")
    slot_row = torch.empty(n_slots, dtype=torch.int32, device=dev)
    send_slot = torch.empty(n_slots, dtype=torch.int32, device=dev)
    _lib.check(L.halo_route_place_send(_lib.ptr(idx), _lib.c_ll(n_slots), _lib.c_int(n_experts), _lib.ptr(block_hist),
                                       _lib.ptr(dst_base), _lib.ptr(slot_row), _lib.ptr(my_prefix), _lib.ptr(send_slot), s),
               "halo_route_place_send")
    max_units = n_slots // 128 + 2 * n_experts + 2
    units = torch.empty(max_units * int(L.halo_moe_push_unit_bytes()), dtype=torch.uint8, device=dev)
    _lib.check(L.halo_moe_plan_push(_lib.ptr(counts), _lib.ptr(dst_base), _lib.ptr(my_prefix), _lib.c_int(me),
                                    _lib.c_int(n_ranks), _lib.c_int(n_experts), _lib.c_int(capacity), _lib.ptr(units),
                                    _lib.ptr(n_units), _lib.c_int(max_units), s), "halo_moe_plan_push")
    max_tiles = capacity // 128
    tiles = torch.empty(max(max_tiles, 1) * int(L.halo_moe_tile_bytes()), dtype=torch.uint8, device=dev)
    _lib.check(L.halo_moe_plan_tiles(ctrl, _lib.c_int(me), _lib.c_int(n_ranks), _lib.c_int(n_experts), _lib.c_int(seq),
                                     _lib.ptr(seg_start), _lib.ptr(seg_rows), _lib.ptr(tiles), _lib.ptr(n_tiles),
                                     _lib.c_int(max_tiles), s), "halo_moe_plan_tiles")
    return RoutingState(n_tokens=T, top_k=k, n_experts=n_experts, n_local=n_local, capacity=capacity, topk_idx=idx,
                        slot_row=slot_row, seg_start=seg_start, seg_rows=seg_rows, total_rows=total_rows, counts=counts,
                        send_slot=send_slot, units=units, n_units=n_units, tiles=tiles, n_tiles=n_tiles, seq=seq)


def _ep_list(state: RoutingState, gated: int, n_cols: int, k_dim: int, b_mn_stride: int, b_k_stride: int, swiglu_f: int = 0):
    """Tile list of one grouped product over the receive-buffer tiles in arrival order (cached per routing state)."""
    key = ("ep", gated, n_cols, k_dim, b_mn_stride, b_k_stride, swiglu_f)
    hit = state.lists.get(key)
    if hit is not None:
        return hit
    L = _lib.lib()
    dev = state.slot_row.device
    tile_n = 128 if swiglu_f else 256
    width = swiglu_f if swiglu_f else n_cols
    max_items = max(state.capacity // 128, 1) * ((width + tile_n - 1) // tile_n)
    lst = torch.empty(max_items * _work_bytes(), dtype=torch.uint8, device=dev)
    count = torch.empty(1, dtype=torch.int32, device=dev)
    _lib.check(L.halo_moe_plan_items(_lib.ptr(state.tiles), _lib.ptr(state.n_tiles), _lib.c_int(n_cols), _lib.c_int(k_dim),
                                     _lib.c_int(b_mn_stride), _lib.c_int(b_k_stride), _lib.c_int(swiglu_f), _lib.c_int(gated),
                                     _lib.ptr(lst), _lib.ptr(count), _lib.c_int(max_items), _lib.stream_ptr(dev)),
               "halo_moe_plan_items")
    state.lists[key] = (lst, count, (width + tile_n - 1) // tile_n)
    return state.lists[key]


def _dispatch_gemm(transport, state: RoutingState, seq: int, x, slot_w, recv, meta, row_w, b2d, c, aux, b_mn: int, epi: int,
                   swiglu_f: int, lst_cnt):
    """Kernel A: this rank's rows of ``x`` go to their owners' ``recv`` buffers while the tiles of this rank's own
    ``recv`` are multiplied with the expert bank ``b2d`` as they fill up."""
    lst, cnt, tiles_n = lst_cnt
    dev = x.device
    H = x.shape[1]
    _lib.check(_lib.lib().halo_moe_dispatch_gemm(
        _lib.ptr(x), _lib.ptr(state.send_slot), _lib.ptr(state.units), _lib.ptr(state.n_units), _lib.ptr(slot_w),
        transport.peer_table(recv), transport.peer_table(meta), transport.peer_table(row_w) if row_w is not None else None,
        transport.arrive_table(seq), _lib.c_int(transport.n_ranks), _lib.c_int(transport.rank), _lib.c_int(H),
        _lib.c_int(state.top_k), _lib.ptr(recv), _lib.c_ll(recv.shape[0]), _lib.ptr(b2d), _lib.c_ll(b2d.shape[0]),
        _lib.c_ll(b2d.shape[1]), _lib.c_ll(b2d.stride(0)), _lib.ptr(c), _lib.ptr(aux), _lib.c_ll(c.stride(0)),
        _lib.c_ll(aux.stride(0) if aux is not None else 0), _lib.c_int(b_mn), _lib.c_int(epi), _lib.c_int(swiglu_f),
        _lib.c_int(tiles_n), _lib.ptr(lst), _lib.ptr(cnt), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)),
        "halo_moe_dispatch_gemm")


def _gemm_combine(transport, a, b2d, slots, meta, b_mn: int, lst_cnt):
    """Kernel B: grouped product of the local rows ``a`` with the expert bank, each output row stored into the slot
    buffer of the rank that owns the token."""
    lst, cnt, tiles_n = lst_cnt
    dev = a.device
    _lib.check(_lib.lib().halo_moe_gemm_combine(
        _lib.ptr(a), _lib.c_ll(a.shape[0]), _lib.c_ll(a.shape[1]), _lib.c_ll(a.stride(0)), _lib.ptr(b2d),
        _lib.c_ll(b2d.shape[0]), _lib.c_ll(b2d.shape[1]), _lib.c_ll(b2d.stride(0)), transport.peer_table(slots), _lib.ptr(meta),
        _lib.c_int(transport.n_ranks), _lib.c_ll(slots.stride(0)), _lib.c_int(b_mn), _lib.c_int(tiles_n), _lib.ptr(lst),
        _lib.ptr(cnt), _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)), "halo_moe_gemm_combine")


def _zero_pads(state: RoutingState, buf, meta, row_w):
    dev = buf.device
    _lib.check(_lib.lib().halo_moe_zero_pads(_lib.ptr(buf), _lib.ptr(meta), _lib.ptr(row_w), _lib.ptr(state.seg_start),
                                             _lib.ptr(state.seg_rows), _lib.c_int(state.n_local), _lib.c_int(buf.shape[1]),
                                             _lib.c_int(state.capacity), _lib.stream_ptr(dev)), "halo_moe_zero_pads")


def _slot_sum(state: RoutingState, slots, w32, out):
    T, k = state.n_tokens, state.top_k
    dev = out.device
    _lib.check(_lib.lib().halo_moe_slot_sum(_lib.ptr(slots), _lib.ptr(state.slot_row), _lib.ptr(w32), _lib.ptr(out), _lib.c_ll(T),
                                            _lib.c_int(k), _lib.c_int(out.shape[1]), _lib.c_int(state.capacity),
                                            _lib.stream_ptr(dev)), "halo_moe_slot_sum")


def _fused_forward(ctx, x, topk_idx, topk_w, w_gate_up, w_down, transport, state_out, grad_mode, skip_output):
    T, H = x.shape
    E_local, F2, _ = w_gate_up.shape
    F = F2 // 2
    n_experts = E_local * transport.n_ranks
    k = topk_idx.shape[1]
    dev = x.device
    _mark("start", dev)
    state = plan_routing_fused(topk_idx, n_experts, transport)
    cap = state.capacity
    recv_x = transport.buffer("recv_x", cap, H, torch.bfloat16, dev)
    meta = transport.buffer("row_meta", cap, 1, torch.int32, dev)
    _zero_pads(state, recv_x, meta, None)
    need_grad = grad_mode and any(ctx.needs_input_grad)
    act = _alloc(transport, (cap, F), torch.bfloat16, dev)
    pre = _alloc(transport, (cap, F2), torch.bfloat16, dev) if need_grad else None
    lst1 = _ep_list(state, 1, F2, H, F2, 0, F)
    _mark("fwd: counts, handshake, plans", dev)
    _dispatch_gemm(transport, state, state.seq, x, None, recv_x, meta, None, w_gate_up.reshape(E_local * F2, H), act, pre, 0,
                   EPI_SWIGLU, F, lst1)
    _mark("fwd: dispatch + gate_up GEMM + SwiGLU", dev)
    w32 = topk_w.float().contiguous()
    out = _alloc(transport, tuple(x.shape), x.dtype, dev)
    if not (skip_output and need_grad):
        slots = transport.buffer("slots", T * k, H, torch.bfloat16, dev)
        lst2 = _ep_list(state, 0, H, F, H, 0)
        _gemm_combine(transport, act, w_down.reshape(E_local * H, F), slots, meta, 0, lst2)
        _mark("fwd: down GEMM + combine stores", dev)
        transport.barrier()
        _mark("fwd: barrier", dev)
        _slot_sum(state, slots, w32, out)
        _mark("fwd: slot sum", dev)
    if need_grad:
        if transport.transient_buffers:
            recv_x = recv_x.clone()
        ctx.save_for_backward(recv_x, pre, w32, w_gate_up, w_down)
        ctx.state = state
        ctx.transport = transport
    if state_out is not None:
        state_out.append(state)
    return out


def _fused_backward(ctx, dout):
    recv_x, pre, w32, w_gate_up, w_down = ctx.saved_tensors
    state, transport = ctx.state, ctx.transport
    T, k = state.n_tokens, state.top_k
    E_local, F2, H = w_gate_up.shape
    F = F2 // 2
    cap = state.capacity
    dev = dout.device
    L = _lib.lib()
    s = _lib.stream_ptr(dev)
    dout = dout.contiguous()
    n_ranks, me = transport.n_ranks, transport.rank
    _mark("start", dev)
    # 1. a handshake of its own: every rank is done with the buffers of its previous call, the arrival counters restart
    seq = transport.next_seq()
    _lib.check(L.halo_moe_handshake(transport.ctrl_table(), _lib.c_int(me), _lib.c_int(n_ranks), _lib.c_int(state.n_experts),
                                    _lib.c_int(seq), _lib.c_int(transport.max_tiles), _lib.c_void_p(0), _lib.c_int(cap),
                                    _lib.c_void_p(0), _lib.c_void_p(0), _lib.c_void_p(0), _lib.c_void_p(0), _lib.c_void_p(0),
                                    _lib.ptr(_lib.status_word(dev)), s), "halo_moe_handshake")
    dy = transport.buffer("recv_dy", cap, H, torch.bfloat16, dev)
    row_w = transport.buffer("row_w", cap, 1, torch.float32, dev)
    meta = transport.buffer("row_meta", cap, 1, torch.int32, dev)
    _zero_pads(state, dy, meta, row_w)
    # 2. dout rows (with their routing weights) travel to the experts inside the first product:
    #    dact_u = dout_rows W_down (unscaled activation gradient)
    dact = _alloc(transport, (cap, F), torch.bfloat16, dev)
    lst = _ep_list(state, 1, F, H, 0, H)
    _mark("bwd: handshake, plans", dev)
    _dispatch_gemm(transport, state, seq, dout, w32, dy, meta, row_w, w_down.reshape(E_local * H, F), dact, None, 1,
                   EPI_STORE_BF16, 0, lst)
    _mark("bwd: dispatch + dact GEMM", dev)
    # 3. SwiGLU backward with the routing weight folded in (dpre over pre, w * act over dact_u); every row's routing-weight
    #    gradient goes straight to the token's owner
    dw_slots = transport.buffer("dw_slots", T * k, 1, torch.float32, dev)
    dpre, act_w = pre, dact
    _lib.check(L.halo_moe_swiglu_bwd_scatter(_lib.ptr(pre), _lib.ptr(dact), _lib.ptr(row_w), _lib.ptr(dpre), _lib.ptr(act_w),
                                             _lib.ptr(meta), transport.peer_table(dw_slots), _lib.c_int(n_ranks),
                                             _lib.ptr(state.total_rows), _lib.c_int(F), _lib.c_int(cap), s),
               "halo_moe_swiglu_bwd_scatter")
    _mark("bwd: SwiGLU backward", dev)
    # 4. input-gradient rows dx_rows = dpre W_gate_up, stored straight into the token owners' slots
    slots = transport.buffer("slots", T * k, H, torch.bfloat16, dev)
    lst = _ep_list(state, 0, H, F2, 0, F2)
    _gemm_combine(transport, dpre, w_gate_up.reshape(E_local * F2, H), slots, meta, 1, lst)
    _mark("bwd: dx GEMM + combine stores", dev)
    # 5. weight gradients (local): dW_down[e] = dout_e^T (w * act)_e ; dW_gate_up[e] = dpre_e^T x_e
    dw_gate_up = dw_down = None
    if ctx.needs_input_grad[3] or ctx.needs_input_grad[4]:
        dw_down = _alloc(transport, tuple(w_down.shape), w_down.dtype, dev)
        pk = _pair_ok(4096, False)
        _gemm_list(dy, act_w, dw_down.reshape(E_local * H, F), _tile_list(state, "k", pk, m_dim=H, n_dim=F), 1, 1,
                   EPI_STORE_BF16, pair=pk)
        dw_gate_up = _alloc(transport, tuple(w_gate_up.shape), w_gate_up.dtype, dev)
        _gemm_list(dpre, recv_x, dw_gate_up.reshape(E_local * F2, H), _tile_list(state, "k", pk, m_dim=F2, n_dim=H), 1, 1,
                   EPI_STORE_BF16, pair=pk)
    _mark("bwd: two weight-gradient GEMMs", dev)
    # 6. every rank's rows have landed: sum the k slots of each token
    transport.barrier()
    _mark("bwd: barrier", dev)
    dx = _alloc(transport, (T, H), torch.bfloat16, dev)
    _slot_sum(state, slots, None, dx)
    _mark("bwd: slot sum", dev)
    # slots of dropped rows (a capacity overflow, reported through the status word) carry no gradient
    valid = (state.slot_row >= 0) & (state.slot_row < cap // 128 * 128)
    dw = torch.where(valid, dw_slots[:T * k, 0], torch.zeros((), dtype=torch.float32, device=dev)).view(T, k)
    return dx, None, dw, dw_gate_up, dw_down, None, None, None, None, None, None, None, None


# ---------------------------------------------------------------------------------------------
# CPU / oracle implementation of the whole routed FFN (also the gloo-rank path)
# ---------------------------------------------------------------------------------------------
def moe_ffn_reference(x, topk_idx, topk_w, w_gate_up, w_down, expert_offset: int = 0):
    """Loop over experts in fp32-accumulate PyTorch. Only experts in
    [expert_offset, expert_offset + E_local) are applied (the rest contribute zero)."""
    T, H = x.shape
    E_local, F2, _ = w_gate_up.shape
    F = F2 // 2
    out = torch.zeros((T, H), dtype=torch.float32, device=x.device)
    for le in range(E_local):
        e = le + expert_offset
        tok, slot = torch.where(topk_idx == e)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        pre = (xe.float() @ w_gate_up[le].float().t()).to(x.dtype)
        act = (torch.nn.functional.silu(pre[:, :F].float()) * pre[:, F:].float()).to(x.dtype)
        ye = (act.float() @ w_down[le].float().t()).to(x.dtype)
        out.index_add_(0, tok, ye.float() * topk_w[tok, slot].float()[:, None])
    return out.to(x.dtype)


# ---------------------------------------------------------------------------------------------
# the fused autograd node
# ---------------------------------------------------------------------------------------------
class _MoEExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topk_idx, topk_w, w_gate_up, w_down, transport, state_out, grad_mode, skip_output=False,
                gate_up_bias=None, down_bias=None, glu_limit=0.0, glu_alpha=0.0):
        # experts with bias vectors / a clamped GLU take the separate-kernel pipeline: their element-wise half runs as
        # row kernels between the grouped products
        ctx.glu = (float(glu_limit), float(glu_alpha)) if gate_up_bias is not None else None
        ctx.fused = _fused(transport) and ctx.glu is None
        if ctx.fused:
            return _fused_forward(ctx, x, topk_idx, topk_w, w_gate_up, w_down, transport, state_out, grad_mode, skip_output)
        T, H = x.shape
        E_local, F2, _ = w_gate_up.shape
        F = F2 // 2
        n_experts = E_local * transport.n_ranks
        k = topk_idx.shape[1]
        dev = x.device
        L = _lib.lib()
        s = _lib.stream_ptr(dev)
        state = plan_routing(topk_idx, n_experts, transport)
        cap = state.capacity
        recv_x = transport.buffer("recv_x", cap, H, torch.bfloat16, dev)
        y_rows = transport.buffer("y_rows", cap, H, torch.bfloat16, dev)
        px = transport.peer_table(recv_x)
        py = transport.peer_table(y_rows)
        _lib.check(L.halo_zero_pad_rows(_lib.ptr(recv_x), _lib.ptr(state.seg_start), _lib.ptr(state.seg_rows),
                                        _lib.c_int(state.n_local), _lib.c_int(H), _lib.c_int(cap), s), "halo_zero_pad_rows")
        transport.barrier_before_push()     # after the local zeroing, before anyone's rows arrive
        _lib.check(L.halo_dispatch_rows(_lib.ptr(x), _lib.ptr(state.topk_idx), _lib.ptr(state.slot_row),
                                        _lib.c_void_p(0), px, _lib.c_void_p(0), _lib.c_int(transport.n_ranks), _lib.c_ll(T), _lib.c_int(k),
                                        _lib.c_int(H), _lib.c_int(E_local), _lib.c_int(cap),
                                        _lib.ptr(_lib.status_word(dev)), s), "halo_dispatch_rows")
        transport.barrier()
        need_grad = grad_mode and any(ctx.needs_input_grad)
        if ctx.glu is None:
            act, pre = grouped_swiglu_ffn_fwd(state, recv_x, w_gate_up, w_down, save_pre=need_grad, transport=transport)
        else:
            act, pre = grouped_biased_glu_fwd(state, recv_x, w_gate_up, gate_up_bias, *ctx.glu, transport=transport)
        w32 = topk_w.float().contiguous()
        if skip_output and need_grad:
            # a recomputation whose value nobody reads: the backward needs only the dispatched rows and the
            # pre-activations, so the down projection and the pull back to the tokens are left out
            out = _alloc(transport, tuple(x.shape), x.dtype, dev)
        else:
            grouped_down_fwd(state, act, w_down, y_rows)
            if ctx.glu is not None:
                _lib.check(L.halo_expert_add_bias_rows(_lib.ptr(y_rows), _lib.ptr(down_bias), _lib.ptr(state.seg_start),
                                                       _lib.c_int(state.n_local), _lib.ptr(state.total_rows), _lib.c_int(H),
                                                       _lib.c_int(cap), s), "halo_expert_add_bias_rows")
            transport.barrier()
            out = _alloc(transport, tuple(x.shape), x.dtype, dev)
            _lib.check(L.halo_combine_rows(py, _lib.c_int(transport.n_ranks), _lib.ptr(state.topk_idx), _lib.ptr(state.slot_row),
                                           _lib.ptr(w32), _lib.c_void_p(0), _lib.ptr(out), _lib.c_ll(T), _lib.c_int(k),
                                           _lib.c_int(H), _lib.c_int(E_local), _lib.c_int(cap), s), "halo_combine_rows")
        if need_grad:
            if transport.transient_buffers:
                recv_x = recv_x.clone()
            ctx.save_for_backward(recv_x, pre, w32, w_gate_up, w_down, down_bias)
            ctx.state = state
            ctx.transport = transport
        if state_out is not None:
            state_out.append(state)
        return out

    @staticmethod
    def backward(ctx, dout):
        if ctx.fused:
            return _fused_backward(ctx, dout)
        recv_x, pre, w32, w_gate_up, w_down, down_bias = ctx.saved_tensors
        state, transport = ctx.state, ctx.transport
        T, k = state.n_tokens, state.top_k
        E_local, F2, H = w_gate_up.shape
        F = F2 // 2
        cap = state.capacity
        dev = dout.device
        L = _lib.lib()
        s = _lib.stream_ptr(dev)
        dout = dout.contiguous()
        # 1. push dout rows (unscaled) and routing weights to the experts
        dy = transport.buffer("recv_dy", cap, H, torch.bfloat16, dev)
        row_w = transport.buffer("row_w", cap, 1, torch.float32, dev)
        row_w.zero_()  # pad rows scale to zero
        pdy, pw = transport.peer_table(dy), transport.peer_table(row_w)
        _lib.check(L.halo_zero_pad_rows(_lib.ptr(dy), _lib.ptr(state.seg_start), _lib.ptr(state.seg_rows),
                                        _lib.c_int(state.n_local), _lib.c_int(H), _lib.c_int(cap), s), "halo_zero_pad_rows")
        transport.barrier_before_push()     # row_w is zeroed everywhere before any rank's weights land in it
        _lib.check(L.halo_dispatch_rows(_lib.ptr(dout), _lib.ptr(state.topk_idx), _lib.ptr(state.slot_row),
                                        _lib.ptr(w32), pdy, pw, _lib.c_int(transport.n_ranks), _lib.c_ll(T), _lib.c_int(k),
                                        _lib.c_int(H), _lib.c_int(E_local), _lib.c_int(cap),
                                        _lib.ptr(_lib.status_word(dev)), s), "halo_dispatch_rows")
        transport.barrier()
        # 2. unscaled activation gradient: dact_u = dout_rows W_down
        dact = _alloc(transport, (cap, F), torch.bfloat16, dev)
        pair = _pair_ok(H, False)
        lst = _tile_list(state, "m", pair, n_cols=F, k_dim=H, b_mn_stride=0, b_k_stride=H, swiglu_f=0)
        _gemm_list(dy, w_down.reshape(E_local * H, F), dact, lst, 0, 1, EPI_STORE_BF16, pair=pair)
        # 3. SwiGLU backward with the routing weight folded in: dpre = w * swiglu'(pre) dact_u, act_w = w * act,
        #    dwrow = <dact_u, act> (= <dout, expert output>, without ever forming the expert output).
        #    Both outputs overwrite their inputs (element for element, same index): dpre lands on pre, act_w on dact_u.
        dwrow = transport.buffer("dwrow", cap, 1, torch.float32, dev)
        dpre, act_w = pre, dact
        d_gate_up_bias = d_down_bias = None
        if ctx.glu is None:
            _lib.check(L.halo_swiglu_bwd_weighted(_lib.ptr(pre), _lib.ptr(dact), _lib.ptr(row_w), _lib.ptr(dpre),
                                                  _lib.ptr(act_w), _lib.ptr(dwrow), _lib.ptr(state.total_rows),
                                                  _lib.c_int(F), _lib.c_int(cap), s), "halo_swiglu_bwd_weighted")
        else:
            limit, alpha = ctx.glu
            _lib.check(L.halo_expert_glu_bwd(_lib.ptr(pre), _lib.ptr(dact), _lib.ptr(row_w), _lib.ptr(dpre), _lib.ptr(act_w),
                                             _lib.ptr(dwrow), _lib.ptr(state.total_rows), _lib.c_int(F), _lib.c_int(cap),
                                             _lib.c_float(limit), _lib.c_float(alpha), s), "halo_expert_glu_bwd")
            # the expert's output includes its down bias: <dout, b_down[e]> joins the routing-weight gradient
            _lib.check(L.halo_expert_bias_rowdot(_lib.ptr(dy), _lib.ptr(down_bias), _lib.ptr(dwrow), _lib.ptr(state.seg_start),
                                                 _lib.c_int(state.n_local), _lib.ptr(state.total_rows), _lib.c_int(H),
                                                 _lib.c_int(cap), s), "halo_expert_bias_rowdot")
            # bias gradients: column sums over each expert's rows (dy is still the incoming gradient here; its storage
            # may take the input-gradient rows below)
            if ctx.needs_input_grad[10]:
                d_down_bias = _expert_colsum(state, dy, row_w, H).to(down_bias.dtype)
            if ctx.needs_input_grad[9]:
                d_gate_up_bias = _expert_colsum(state, dpre, None, F2).to(down_bias.dtype)
        need_weight_grads = ctx.needs_input_grad[3] or ctx.needs_input_grad[4]

        def weight_grads():
            if not need_weight_grads:      # frozen banks (adapters elsewhere): the two products are left out
                return None, None
            # 5. dW_down[e] = dout_e^T (w * act)_e ; dW_gate_up[e] = dpre_e^T x_e
            dw_down = _alloc(transport, tuple(w_down.shape), w_down.dtype, dev)
            pk = _pair_ok(4096, False)      # the reduction runs over an expert's rows: long
            _gemm_list(dy, act_w, dw_down.reshape(E_local * H, F), _tile_list(state, "k", pk, m_dim=H, n_dim=F), 1, 1,
                       EPI_STORE_BF16, pair=pk)
            dw_gate_up = _alloc(transport, tuple(w_gate_up.shape), w_gate_up.dtype, dev)
            _gemm_list(dpre, recv_x, dw_gate_up.reshape(E_local * F2, H), _tile_list(state, "k", pk, m_dim=F2, n_dim=H), 1, 1,
                       EPI_STORE_BF16, pair=pk)
            return dw_gate_up, dw_down

        # 4. input gradient rows: dx_rows = dpre W_gate_up. On one rank the weight gradients go first, after which the
        #    incoming-gradient rows are dead and their storage takes dx_rows; across ranks dx_rows is the peers' window
        #    and goes first so that its pull can run beside the weight gradients.
        early_weight_grads = transport.n_ranks == 1
        if early_weight_grads:
            dw_gate_up, dw_down = weight_grads()
            dx_rows = dy
        else:
            dx_rows = transport.buffer("dx_rows", cap, H, torch.bfloat16, dev)
        pair = _pair_ok(F2, False)
        lst = _tile_list(state, "m", pair, n_cols=H, k_dim=F2, b_mn_stride=0, b_k_stride=F2, swiglu_f=0)
        _gemm_list(dpre, w_gate_up.reshape(E_local * F2, H), dx_rows, lst, 0, 1, EPI_STORE_BF16, pair=pair)
        dx = _alloc(transport, (T, H), torch.bfloat16, dev)
        dw = _alloc(transport, (T, k), torch.float32, dev)
        pdx, pdw = transport.peer_table(dx_rows), transport.peer_table(dwrow)

        def pull_back():
            # 6. pull the input-gradient rows and the routing-weight gradients back to the tokens
            st = _lib.stream_ptr(dev)
            _lib.check(L.halo_combine_rows(pdx, _lib.c_int(transport.n_ranks), _lib.ptr(state.topk_idx), _lib.ptr(state.slot_row),
                                           _lib.c_void_p(0), _lib.c_void_p(0), _lib.ptr(dx), _lib.c_ll(T), _lib.c_int(k),
                                           _lib.c_int(H), _lib.c_int(E_local), _lib.c_int(cap), st), "halo_combine_rows")
            _lib.check(L.halo_gather_slot_values(pdw, _lib.c_int(transport.n_ranks), _lib.ptr(state.topk_idx), _lib.ptr(state.slot_row),
                                                 _lib.ptr(dw), _lib.c_ll(T * k), _lib.c_int(E_local), _lib.c_int(cap), st),
                       "halo_gather_slot_values")

        side = transport.side_stream(dev) if transport.n_ranks > 1 else None
        if side is None:
            if not early_weight_grads:
                dw_gate_up, dw_down = weight_grads()
            transport.barrier()
            pull_back()
        else:
            # the pull over NVLink runs beside the two weight-gradient products, which need nothing from it
            main = torch.cuda.current_stream(dev)
            fork = torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                transport.barrier(channel=1)
                pull_back()
                joined = torch.cuda.Event()
                joined.record(side)
            dw_gate_up, dw_down = weight_grads()
            main.wait_event(joined)
        return dx, None, dw, dw_gate_up, dw_down, None, None, None, None, d_gate_up_bias, d_down_bias, None, None


def _moe_experts_lanes(x, topk_idx, topk_w, w_gate_up, w_down, lanes, state_out, skip_output, glu=(None, None, 0.0, 0.0)):
    """Cut the tokens into one part per lane and run each part's whole expert op (push, products, pull) on the
    lane's own stream and buffers: while one part moves rows over NVLink, another part's products keep the
    tensor cores busy. Every rank cuts at the same places, so the lanes' barriers pair up across ranks."""
    T = x.shape[0]
    n = len(lanes) if T >= 256 * len(lanes) else 1
    step = ((T + n - 1) // n + 127) // 128 * 128
    dev = x.device
    main = torch.cuda.current_stream(dev)
    fork = torch.cuda.Event()
    fork.record(main)
    grad_mode = torch.is_grad_enabled()
    outs, done = [], []
    for i in range(n):
        lo, hi = i * step, min(T, (i + 1) * step)
        if lo >= hi:
            break
        lane = lanes[i]
        lane.alloc_stream = main
        xs, ids, ws = x[lo:hi], topk_idx[lo:hi], topk_w[lo:hi]
        lane.stream.wait_event(fork)
        with torch.cuda.stream(lane.stream):
            o = _MoEExperts.apply(xs, ids, ws, w_gate_up, w_down, lane, state_out, grad_mode, skip_output, *glu)
            ev = torch.cuda.Event()
            ev.record(lane.stream)
        outs.append(o)
        done.append(ev)
    for ev in done:
        main.wait_event(ev)
    for o in outs:
        o.record_stream(main)
    return outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)


def moe_experts(x, topk_idx, topk_w, w_gate_up, w_down, transport=None, state_out: list | None = None,
                skip_output: bool = False, glu: tuple | None = None):
    """Apply the routed experts.

    x: [T, H] bf16; topk_idx: int32 [T, k] global expert ids; topk_w: [T, k] routing weights;
    w_gate_up: [E_local, 2F, H] (gate rows then up rows per expert); w_down: [E_local, H, F].
    ``skip_output``: the caller will not read the result (a recomputation that only rebuilds what the
    backward needs); the returned tensor is then uninitialised.
    ``glu = (gate_up_bias [E_local, 2F], down_bias [E_local, H], limit, alpha)``: experts with bias vectors around a
    clamped GLU, ``(up + 1) * gate * sigmoid(alpha * gate)`` with ``gate <= limit`` and ``|up| <= limit`` (GPU only: the
    tensor-op form is :func:`halo_b200.ops.biased_glu_experts.biased_glu_experts`).
    """
    if transport is None:
        transport = LocalTransport()
    if glu is not None:
        if not x.is_cuda or not hasattr(transport, "peer_table"):
            raise NotImplementedError("experts with bias vectors / a clamped GLU run through the grouped kernels on a GPU only")
        glu = (glu[0].contiguous(), glu[1].contiguous(), float(glu[2]), float(glu[3]))
    if not x.is_cuda or hasattr(transport, "reference_ffn") and not hasattr(transport, "peer_table"):
        offset = transport.rank * w_gate_up.shape[0]
        if transport.n_ranks > 1:
            return transport.reference_ffn(x, topk_idx, topk_w, w_gate_up, w_down)
        return moe_ffn_reference(x, topk_idx, topk_w, w_gate_up, w_down, offset)
    lanes = getattr(transport, "lanes", None)
    extra = glu if glu is not None else (None, None, 0.0, 0.0)
    if lanes:
        return _moe_experts_lanes(x.contiguous(), topk_idx, topk_w, w_gate_up, w_down, lanes, state_out, skip_output, extra)
    return _MoEExperts.apply(x.contiguous(), topk_idx, topk_w, w_gate_up, w_down, transport, state_out,
                             torch.is_grad_enabled(), skip_output, *extra)
