"""Residual-stream ops of the hyper-connected and gated-residual decoder families.

``N`` parallel residual streams ``[..., N, H]`` replace the single residual: before a block they are *collapsed*
into one input with per-token weights, after it the block's output is *mixed* back (``post`` weights the new
output per stream, a doubly-stochastic ``comb`` matrix - the Sinkhorn-Knopp projection of per-token logits -
mixes the old streams), or simply *injected* with a gate. The weights come from a *projection* of the RMS-scaled
flattened streams. The gated-residual family adds a per-stream RMSNorm with ``(1 + w)`` scaling and a
sigmoid-gated mean over streams.

Every op is an autograd function with a closed-form backward. bf16 CUDA tensors run the sm_100a kernels of
``csrc/streams.cu`` (one pass over the streams each way, fp32 math, one rounding at the store); anything else runs
the same formulas in PyTorch, and the ``*_reference`` functions state each op as the plain differentiable
expression the tests compare against.

Behavioural counterparts: halo/kernels/hyper_connection.py:209-630, halo/kernels/gated_residual.py:148-200,
halo/kernels/masked_softmax.py:46-77.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

MAX_STREAMS = 8


# ---- plain expressions (oracles) -------------------------------------------------------------------------------
def project_streams_reference(stream, fn, norm_eps):
    x = stream.flatten(-2).float()
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + norm_eps)
    return F.linear(x, fn.float())


def sinkhorn_knopp_reference(comb, iters, eps):
    m = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(iters - 1):
        m = m / (m.sum(-1, keepdim=True) + eps)
        m = m / (m.sum(-2, keepdim=True) + eps)
    return m


def collapse_streams_reference(stream, weight):
    return (weight.unsqueeze(-1).float() * stream.float()).sum(-2).to(stream.dtype)


def mix_streams_reference(block, residual, post, comb):
    out = post.unsqueeze(-1).float() * block.unsqueeze(-2).float() + comb.transpose(-1, -2).float() @ residual.float()
    return out.to(residual.dtype)


def inject_streams_reference(block, residual, gate):
    return (residual.float() + gate.unsqueeze(-1).float() * block.unsqueeze(-2).float()).to(residual.dtype)


def grouped_rms_norm_reference(x, weight, eps, streams):
    rows, width = x.shape
    g = x.float().view(rows, streams, width // streams)
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    return (g.view(rows, width) * (1.0 + weight.float())).to(x.dtype)


def gate_mix_reference(normed, down, w_up, streams):
    rows = normed.shape[0]
    up = F.linear(F.silu(down / streams), w_up)
    return (torch.sigmoid(up) * normed).view(rows, streams, -1).mean(-2)


# ---- dispatch helpers ---------------------------------------------------------------------------------------------
def _on_kernels(*tensors) -> bool:
    """bf16 CUDA tensors whose rows are whole 16-byte vectors starting on a 16-byte boundary."""
    return all(t.is_cuda and t.dtype == torch.bfloat16 and t.shape[-1] % 8 == 0 and t.data_ptr() % 16 == 0 for t in tensors)


def _check_streams(n: int) -> None:
    if not 1 <= n <= MAX_STREAMS:
        raise ValueError(f"{n} residual streams: the stream ops are built for 1..{MAX_STREAMS}")


def _require(tensor, shape, name):
    if tuple(tensor.shape) != tuple(shape):
        raise ValueError(f"{name} of shape {tuple(tensor.shape)} where the streams take {tuple(shape)}")


def _f32(t):
    return t.detach().float().contiguous()


# ---- collapse ------------------------------------------------------------------------------------------------------
class _Collapse(torch.autograd.Function):
    @staticmethod
    def forward(ctx, stream, weight):
        lead, (N, H) = stream.shape[:-2], stream.shape[-2:]
        x = stream.reshape(-1, N, H).contiguous()
        w = _f32(weight.reshape(-1, N))
        T = x.shape[0]
        if _on_kernels(x):
            out = torch.empty((T, H), dtype=x.dtype, device=x.device)
            _lib.check(_lib.lib().halo_stream_collapse_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(out), _lib.c_ll(T), _lib.c_int(N),
                                                           _lib.c_int(H), _lib.stream_ptr(x.device)), "halo_stream_collapse_fwd")
        else:
            out = (w.unsqueeze(-1) * x.float()).sum(-2).to(x.dtype)
        ctx.save_for_backward(x, w)
        ctx.meta = (lead, N, H, weight.dtype)
        return out.reshape(*lead, H)

    @staticmethod
    def backward(ctx, grad_out):
        x, w = ctx.saved_tensors
        lead, N, H, w_dtype = ctx.meta
        T = x.shape[0]
        g = grad_out.reshape(T, H).contiguous()
        if _on_kernels(x, g):
            dx = torch.empty_like(x)
            dw = torch.empty((T, N), dtype=torch.float32, device=x.device)
            _lib.check(_lib.lib().halo_stream_collapse_bwd(_lib.ptr(g), _lib.ptr(x), _lib.ptr(w), _lib.ptr(dx), _lib.ptr(dw),
                                                           _lib.c_ll(T), _lib.c_int(N), _lib.c_int(H), _lib.stream_ptr(x.device)),
                       "halo_stream_collapse_bwd")
        else:
            gf = g.float()
            dx = (w.unsqueeze(-1) * gf.unsqueeze(-2)).to(x.dtype)
            dw = (gf.unsqueeze(-2) * x.float()).sum(-1)
        return dx.reshape(*lead, N, H), dw.to(w_dtype).reshape(*lead, N)


def collapse_streams(stream: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``(weight.unsqueeze(-1) * stream).sum(-2)`` for ``[..., N, H]`` streams and ``[..., N]`` weights, computed in
    fp32 and stored in the streams' dtype."""
    _check_streams(stream.shape[-2])
    _require(weight, stream.shape[:-1], "weight")
    return _Collapse.apply(stream, weight)


# ---- mix -----------------------------------------------------------------------------------------------------------
class _Mix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, block, residual, post, comb):
        lead, (N, H) = residual.shape[:-2], residual.shape[-2:]
        b = block.reshape(-1, H).contiguous()
        r = residual.reshape(-1, N, H).contiguous()
        p, c = _f32(post.reshape(-1, N)), _f32(comb.reshape(-1, N, N))
        T = r.shape[0]
        if _on_kernels(r, b):
            out = torch.empty_like(r)
            _lib.check(_lib.lib().halo_stream_mix_fwd(_lib.ptr(b), _lib.ptr(r), _lib.ptr(p), _lib.ptr(c), _lib.ptr(out), _lib.c_ll(T),
                                                      _lib.c_int(N), _lib.c_int(H), _lib.stream_ptr(r.device)), "halo_stream_mix_fwd")
        else:
            out = (p.unsqueeze(-1) * b.float().unsqueeze(-2) + c.transpose(-1, -2) @ r.float()).to(r.dtype)
        ctx.save_for_backward(b, r, p, c)
        ctx.meta = (lead, N, H, post.dtype, comb.dtype)
        return out.reshape(*lead, N, H)

    @staticmethod
    def backward(ctx, grad_out):
        b, r, p, c = ctx.saved_tensors
        lead, N, H, p_dtype, c_dtype = ctx.meta
        T = r.shape[0]
        g = grad_out.reshape(T, N, H).contiguous()
        if _on_kernels(r, b, g):
            db, dr = torch.empty_like(b), torch.empty_like(r)
            dp = torch.empty((T, N), dtype=torch.float32, device=r.device)
            dc = torch.empty((T, N, N), dtype=torch.float32, device=r.device)
            _lib.check(_lib.lib().halo_stream_mix_bwd(_lib.ptr(g), _lib.ptr(b), _lib.ptr(r), _lib.ptr(p), _lib.ptr(c), _lib.ptr(db),
                                                      _lib.ptr(dr), _lib.ptr(dp), _lib.ptr(dc), _lib.c_ll(T), _lib.c_int(N),
                                                      _lib.c_int(H), _lib.stream_ptr(r.device)), "halo_stream_mix_bwd")
        else:
            gf, bf, rf = g.float(), b.float(), r.float()
            db = (p.unsqueeze(-1) * gf).sum(-2).to(b.dtype)
            dp = (gf * bf.unsqueeze(-2)).sum(-1)
            dr = (c @ gf).to(r.dtype)                       # dres[n] = sum_m comb[n, m] g[m]
            dc = rf @ gf.transpose(-1, -2)                  # dcomb[n, m] = <res[n], g[m]>
        return db.reshape(*lead, H), dr.reshape(*lead, N, H), dp.to(p_dtype).reshape(*lead, N), dc.to(c_dtype).reshape(*lead, N, N)


def mix_streams(block: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """``post.unsqueeze(-1) * block.unsqueeze(-2) + comb.transpose(-1, -2) @ residual`` for ``[..., H]`` ``block``,
    ``[..., N, H]`` ``residual``, ``[..., N]`` ``post`` and ``[..., N, N]`` ``comb``."""
    N = residual.shape[-2]
    _check_streams(N)
    _require(block, residual.shape[:-2] + residual.shape[-1:], "block")
    _require(post, residual.shape[:-1], "post")
    _require(comb, residual.shape[:-1] + (N,), "comb")
    return _Mix.apply(block, residual, post, comb)


# ---- inject --------------------------------------------------------------------------------------------------------
class _Inject(torch.autograd.Function):
    @staticmethod
    def forward(ctx, block, residual, gate):
        lead, (N, H) = residual.shape[:-2], residual.shape[-2:]
        b = block.reshape(-1, H).contiguous()
        r = residual.reshape(-1, N, H).contiguous()
        gt = _f32(gate.reshape(-1, N))
        T = r.shape[0]
        if _on_kernels(r, b):
            out = torch.empty_like(r)
            _lib.check(_lib.lib().halo_stream_inject_fwd(_lib.ptr(b), _lib.ptr(r), _lib.ptr(gt), _lib.ptr(out), _lib.c_ll(T),
                                                         _lib.c_int(N), _lib.c_int(H), _lib.stream_ptr(r.device)), "halo_stream_inject_fwd")
        else:
            out = (r.float() + gt.unsqueeze(-1) * b.float().unsqueeze(-2)).to(r.dtype)
        ctx.save_for_backward(b, gt)
        ctx.meta = (lead, N, H, gate.dtype)
        return out.reshape(*lead, N, H)

    @staticmethod
    def backward(ctx, grad_out):
        b, gt = ctx.saved_tensors
        lead, N, H, g_dtype = ctx.meta
        T = b.shape[0]
        g = grad_out.reshape(T, N, H).contiguous()
        if _on_kernels(g, b):
            db = torch.empty_like(b)
            dg = torch.empty((T, N), dtype=torch.float32, device=b.device)
            _lib.check(_lib.lib().halo_stream_inject_bwd(_lib.ptr(g), _lib.ptr(b), _lib.ptr(gt), _lib.ptr(db), _lib.ptr(dg), _lib.c_ll(T),
                                                         _lib.c_int(N), _lib.c_int(H), _lib.stream_ptr(b.device)), "halo_stream_inject_bwd")
        else:
            gf = g.float()
            db = (gt.unsqueeze(-1) * gf).sum(-2).to(b.dtype)
            dg = (gf * b.float().unsqueeze(-2)).sum(-1)
        return db.reshape(*lead, H), grad_out, dg.to(g_dtype).reshape(*lead, N)


def inject_streams(block: torch.Tensor, residual: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``residual + gate.unsqueeze(-1) * block.unsqueeze(-2)`` for ``[..., H]`` ``block``, ``[..., N, H]`` ``residual``
    and ``[..., N]`` ``gate``."""
    _check_streams(residual.shape[-2])
    _require(block, residual.shape[:-2] + residual.shape[-1:], "block")
    _require(gate, residual.shape[:-1], "gate")
    return _Inject.apply(block, residual, gate)


# ---- Sinkhorn-Knopp ------------------------------------------------------------------------------------------------
def _sinkhorn_forward(comb, iters, eps, save):
    N = comb.shape[-1]
    c = comb.reshape(-1, N, N).float().contiguous()
    T = c.shape[0]
    steps = 2 * (iters - 1) + 1
    if c.is_cuda:
        out = torch.empty_like(c)
        scales = torch.empty((T, steps, N), dtype=torch.float32, device=c.device) if save else None
        _lib.check(_lib.lib().halo_sinkhorn_fwd(_lib.ptr(c), _lib.ptr(out), _lib.ptr(scales), _lib.c_ll(T), _lib.c_int(N),
                                                _lib.c_int(iters), _lib.c_float(eps), _lib.stream_ptr(c.device)), "halo_sinkhorn_fwd")
        return out, scales
    kept = []
    m = c
    s = m.sum(-2, keepdim=True) + eps
    kept.append(s.squeeze(-2))
    m = m / s
    for _ in range(iters - 1):
        s = m.sum(-1, keepdim=True) + eps
        kept.append(s.squeeze(-1))
        m = m / s
        s = m.sum(-2, keepdim=True) + eps
        kept.append(s.squeeze(-2))
        m = m / s
    return m, (torch.stack(kept, dim=1) if save else None)


class _Sinkhorn(torch.autograd.Function):
    """Keeps the final matrix and every step's divisor ``[T, 2 * iters - 1, N]``: the earlier matrices follow from
    them on the way back."""

    @staticmethod
    def forward(ctx, comb, iters, eps):
        out, scales = _sinkhorn_forward(comb, iters, eps, save=True)
        ctx.save_for_backward(out, scales)
        ctx.meta = (iters, comb.shape, comb.dtype)
        return out.to(comb.dtype).reshape(comb.shape)

    @staticmethod
    def backward(ctx, grad_out):
        out, scales = ctx.saved_tensors
        iters, shape, dtype = ctx.meta
        T, N = out.shape[0], out.shape[-1]
        g = grad_out.reshape(T, N, N).float().contiguous()
        if out.is_cuda:
            dcomb = torch.empty_like(out)
            _lib.check(_lib.lib().halo_sinkhorn_bwd(_lib.ptr(g), _lib.ptr(out), _lib.ptr(scales), _lib.ptr(dcomb), _lib.c_ll(T),
                                                    _lib.c_int(N), _lib.c_int(iters), _lib.stream_ptr(out.device)), "halo_sinkhorn_bwd")
        else:
            y = out

            def reverse(g, y, s, axis):
                s = s.unsqueeze(axis)
                return (g - (g * y).sum(axis, keepdim=True)) / s, y * s

            steps = scales.shape[1]
            for l in range(iters - 1):
                step = steps - 1 - 2 * l
                g, y = reverse(g, y, scales[:, step], -2)
                g, y = reverse(g, y, scales[:, step - 1], -1)
            dcomb, _ = reverse(g, y, scales[:, 0], -2)
        return dcomb.to(dtype).reshape(shape), None, None


def sinkhorn_knopp(comb: torch.Tensor, iters: int, eps: float) -> torch.Tensor:
    """``comb / (comb.sum(-2, keepdim=True) + eps)``, then ``iters - 1`` passes of the same over rows and columns,
    over ``[..., N, N]``. Nothing is kept when no graph is recorded."""
    _check_streams(comb.shape[-1])
    if iters < 1:
        raise ValueError("sinkhorn_knopp needs at least one iteration")
    if torch.is_grad_enabled() and comb.requires_grad:
        return _Sinkhorn.apply(comb, iters, eps)
    return _sinkhorn_forward(comb, iters, eps, save=False)[0].to(comb.dtype).reshape(comb.shape)


# ---- projection of the RMS-scaled flattened streams -----------------------------------------------------------------
class _Project(torch.autograd.Function):
    """``F.linear(x * rstd, fn)`` with fp32 weights on bf16 streams: the product keeps ``x`` in its storage dtype and
    scales the fp32 result by ``rstd`` afterwards (the scale is per row, so it commutes with the product)."""

    @staticmethod
    def forward(ctx, stream, fn, norm_eps):
        lead = stream.shape[:-2]
        W = stream.shape[-2] * stream.shape[-1]
        x = stream.reshape(-1, W).contiguous()
        T = x.shape[0]
        if _on_kernels(x):
            rstd = torch.empty(T, dtype=torch.float32, device=x.device)
            _lib.check(_lib.lib().halo_row_rstd(_lib.ptr(x), _lib.ptr(rstd), _lib.c_ll(T), _lib.c_int(W), _lib.c_float(norm_eps),
                                                _lib.stream_ptr(x.device)), "halo_row_rstd")
        else:
            rstd = torch.rsqrt(x.float().pow(2).mean(-1) + norm_eps)
        raw = _skinny_product(x, fn)                        # [T, K] fp32 = x @ fn^T
        ctx.save_for_backward(x, fn, rstd, raw)
        ctx.lead = lead
        ctx.stream_shape = stream.shape
        return (raw * rstd.unsqueeze(-1)).reshape(*lead, fn.shape[0])

    @staticmethod
    def backward(ctx, grad_out):
        x, fn, rstd, raw = ctx.saved_tensors
        K, W = fn.shape
        g = grad_out.reshape(-1, K).float()
        gs = g * rstd.unsqueeze(-1)                                  # gradient of the raw product
        # y = rstd * raw, rstd = (mean(x^2) + eps)^-1/2:  dx = gs @ fn - x * rstd^2 * sum_k(g * y) / W
        coeff = (g * raw).sum(-1) * rstd.pow(3) / W
        dx = None
        if ctx.needs_input_grad[0]:
            dx = (gs @ fn.float() - x.float() * coeff.unsqueeze(-1)).to(x.dtype).reshape(ctx.stream_shape)
        dfn = None
        if ctx.needs_input_grad[1]:
            if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:
                from .gemm import matmul

                gs16 = _pad_rows(gs.t().contiguous()).t().contiguous().to(x.dtype)        # [T, Kp]: columns padded to 8
                dfn = matmul(gs16, x, a_t=True, b_t=False, out_dtype=torch.float32)[:K]
            else:
                dfn = gs.t() @ x.float()
            dfn = dfn.to(fn.dtype)
        return dx, dfn, None


def _pad_rows(t: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    extra = (-t.shape[0]) % multiple
    return t if not extra else torch.cat([t, t.new_zeros(extra, *t.shape[1:])], dim=0)


def _skinny_product(x: torch.Tensor, fn: torch.Tensor) -> torch.Tensor:
    """``x @ fn^T`` in fp32 for a handful of output columns. On CUDA the fp32 weights are split into a bf16 head
    and a bf16 remainder so the wide bf16 ``x`` is read once by one tensor-core product with an fp32 result; the two
    partial results are added in fp32 (relative error ~2^-16 of the weights, far below the bf16 rounding already in
    ``x``)."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.shape[1] % 8:
        return x.float() @ fn.float().t()
    from .gemm import matmul

    K = fn.shape[0]
    f32 = fn.detach().float()
    hi = f32.to(torch.bfloat16)
    lo = (f32 - hi.float()).to(torch.bfloat16)
    hi, lo = _pad_rows(hi), _pad_rows(lo)                    # the GEMM wants row counts in multiples of 8
    Kp = hi.shape[0]
    out = matmul(x, torch.cat([hi, lo], dim=0), out_dtype=torch.float32)        # [T, 2 Kp] fp32
    return out[:, :K] + out[:, Kp:Kp + K]


def project_streams(stream: torch.Tensor, fn: torch.Tensor, norm_eps: float) -> torch.Tensor:
    """``F.linear(x / rms(x), fn)`` in fp32 with ``x`` the streams of ``[..., N, H]`` flattened per token, where
    ``rms(x) = sqrt(mean(x^2) + norm_eps)`` and ``fn`` is ``[K, N * H]``. Returns ``[..., K]`` fp32."""
    _require(fn, (fn.shape[0], stream.shape[-2] * stream.shape[-1]), "fn")
    return _Project.apply(stream, fn, norm_eps)


# ---- per-stream RMSNorm with (1 + w) ---------------------------------------------------------------------------------
class _GroupedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, streams):
        rows, W = x.shape
        H = W // streams
        x = x.contiguous()
        w = _f32(weight)
        if _on_kernels(x) and H % 8 == 0:
            y = torch.empty_like(x)
            rstd = torch.empty(rows * streams, dtype=torch.float32, device=x.device)
            _lib.check(_lib.lib().halo_grouped_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd), _lib.c_ll(rows),
                                                           _lib.c_int(streams), _lib.c_int(H), _lib.c_float(eps),
                                                           _lib.stream_ptr(x.device)), "halo_grouped_rmsnorm_fwd")
        else:
            g = x.float().view(rows, streams, H)
            rstd = torch.rsqrt(g.pow(2).mean(-1) + eps).reshape(-1)
            y = ((g * rstd.view(rows, streams, 1)).view(rows, W) * (1.0 + w)).to(x.dtype)
        ctx.save_for_backward(x, w, rstd)
        ctx.meta = (streams, H, weight.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        streams, H, w_dtype = ctx.meta
        rows, W = x.shape
        dy = dy.contiguous()
        if _on_kernels(x, dy) and H % 8 == 0:
            L = _lib.lib()
            dx = torch.empty_like(x)
            slabs = L.halo_grouped_rmsnorm_slabs(_lib.c_ll(rows))
            partial = torch.empty((slabs, W), dtype=torch.float32, device=x.device)
            dw = torch.empty(W, dtype=torch.float32, device=x.device)
            _lib.check(L.halo_grouped_rmsnorm_bwd(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(partial),
                                                  _lib.ptr(dw), _lib.c_ll(rows), _lib.c_int(streams), _lib.c_int(H),
                                                  _lib.stream_ptr(x.device)), "halo_grouped_rmsnorm_bwd")
        else:
            g = x.float().view(rows, streams, H)
            r = rstd.view(rows, streams, 1)
            gw = (dy.float() * (1.0 + w)).view(rows, streams, H)
            dot = (gw * g).sum(-1, keepdim=True)
            dx = (r * gw - g * r.pow(3) * dot / H).view(rows, W).to(x.dtype)
            dw = (dy.float().view(rows, streams, H) * g * r).view(rows, W).sum(0)
        return dx, dw.to(w_dtype), None, None


def grouped_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, streams: int) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * (1 + weight)`` per group of ``weight.numel() / streams`` features, for
    ``[rows, streams * hidden]`` ``x`` and a ``[streams * hidden]`` ``weight``; fp32 math, stored in ``x``'s dtype."""
    if x.dim() != 2 or weight.numel() != x.shape[1] or x.shape[1] % streams:
        raise ValueError(f"x {tuple(x.shape)} and weight {tuple(weight.shape)} do not describe {streams} streams")
    return _GroupedRMSNorm.apply(x, weight, eps, streams)


# ---- gated stream mean -----------------------------------------------------------------------------------------------
class _GateMix(torch.autograd.Function):
    """``mean_streams(sigmoid(up) * normed)`` for ``up = Linear(silu(down / N))``: the activation and ``up`` are
    recomputed on the way back, so the graph holds ``normed`` and ``down`` only."""

    @staticmethod
    def _up(down, w_up, streams):
        return F.linear(F.silu(down / streams), w_up)

    @staticmethod
    def forward(ctx, normed, down, w_up, streams):
        rows, W = normed.shape
        H = W // streams
        normed, down, w_up = normed.contiguous(), down.contiguous(), w_up.contiguous()
        up = _GateMix._up(down, w_up, streams)
        if _on_kernels(normed, up) and H % 8 == 0 and streams <= MAX_STREAMS:
            out = torch.empty((rows, H), dtype=normed.dtype, device=normed.device)
            _lib.check(_lib.lib().halo_gate_mix_fwd(_lib.ptr(up), _lib.ptr(normed), _lib.ptr(out), _lib.c_ll(rows), _lib.c_int(streams),
                                                    _lib.c_int(H), _lib.stream_ptr(normed.device)), "halo_gate_mix_fwd")
        else:
            out = (torch.sigmoid(up) * normed).view(rows, streams, H).mean(-2)
        ctx.save_for_backward(normed, down, w_up)
        ctx.streams = streams
        return out

    @staticmethod
    def backward(ctx, dout):
        normed, down, w_up = ctx.saved_tensors
        streams = ctx.streams
        rows, W = normed.shape
        H = W // streams
        dout = dout.contiguous()
        act = F.silu(down / streams)
        up = F.linear(act, w_up)
        if _on_kernels(normed, up, dout) and H % 8 == 0 and streams <= MAX_STREAMS:
            dup, dnormed = torch.empty_like(up), torch.empty_like(normed)
            _lib.check(_lib.lib().halo_gate_mix_bwd(_lib.ptr(dout), _lib.ptr(up), _lib.ptr(normed), _lib.ptr(dup), _lib.ptr(dnormed),
                                                    _lib.c_ll(rows), _lib.c_int(streams), _lib.c_int(H),
                                                    _lib.stream_ptr(normed.device)), "halo_gate_mix_bwd")
        else:
            sg = torch.sigmoid(up.float())
            gd = (dout.float() / streams).unsqueeze(1).expand(rows, streams, H).reshape(rows, W)
            dnormed = (gd * sg).to(normed.dtype)
            dup = (gd * normed.float() * sg * (1.0 - sg)).to(up.dtype)
        dw_up = dup.t() @ act if ctx.needs_input_grad[2] else None
        ddown = None
        if ctx.needs_input_grad[1]:
            dact = (dup @ w_up).float()
            z = down.float() / streams
            s = torch.sigmoid(z)
            ddown = (dact * s * (1.0 + z * (1.0 - s)) / streams).to(down.dtype)
        return dnormed, ddown, dw_up, None


def gate_mix(normed: torch.Tensor, down: torch.Tensor, w_up: torch.Tensor, streams: int) -> torch.Tensor:
    """``(sigmoid(F.linear(silu(down / streams), w_up)) * normed).view(rows, streams, hidden).mean(-2)`` for
    ``[rows, streams * hidden]`` ``normed``, ``[rows, rank]`` ``down`` and a ``[streams * hidden, rank]`` ``w_up``."""
    if w_up.shape[0] != normed.shape[1] or normed.shape[1] % streams or down.shape != (normed.shape[0], w_up.shape[1]):
        raise ValueError(f"normed {tuple(normed.shape)}, down {tuple(down.shape)}, w_up {tuple(w_up.shape)} do not fit {streams} streams")
    return _GateMix.apply(normed, down, w_up, streams)


# ---- masked softmax backward -----------------------------------------------------------------------------------------
def masked_softmax_backward(scores, allowed, lse, scale, upstream_scores=None, delta=None, writes_probs=True,
                            dtype=torch.bfloat16):
    """``probs = exp(scores * scale - lse)`` under the ``[Q, K]`` mask ``allowed`` and, with ``upstream_scores``, the
    softmax's backward onto its scores ``probs * (upstream_scores - delta) * scale``; both ``[H, Q, K]`` in ``dtype``.
    ``scores`` / ``upstream_scores`` are fp32 ``[H, Q, K]``, ``lse`` / ``delta`` ``[H, Q]``. Returns ``(probs | None,
    d_scores | None)``."""
    heads, queries, keys = scores.shape
    want_grad = upstream_scores is not None
    if scores.is_cuda and scores.dtype == torch.float32 and dtype in (torch.bfloat16, torch.float32):
        scores = scores.contiguous()
        if allowed.stride(-1) != 1:
            allowed = allowed.contiguous()
        mask = allowed.view(torch.uint8) if allowed.dtype == torch.bool else allowed.to(torch.uint8)
        probs = torch.empty(scores.shape, dtype=dtype, device=scores.device) if writes_probs else None
        d_scores = torch.empty(scores.shape, dtype=dtype, device=scores.device) if want_grad else None
        up = upstream_scores.float().contiguous() if want_grad else None
        dl = delta.float().contiguous() if want_grad else None
        _lib.check(_lib.lib().halo_masked_softmax_bwd(
            _lib.ptr(scores), _lib.ptr(mask), _lib.ptr(lse.float().contiguous()), _lib.ptr(up), _lib.ptr(dl), _lib.ptr(probs),
            _lib.ptr(d_scores), _lib.c_ll(heads * queries), _lib.c_int(queries), _lib.c_int(keys), _lib.c_ll(mask.stride(0)),
            _lib.c_float(scale), _lib.c_int(1 if dtype == torch.bfloat16 else 0), _lib.stream_ptr(scores.device)),
            "halo_masked_softmax_bwd")
        return probs, d_scores
    p = torch.where(allowed.bool(), torch.exp(scores.float() * scale - lse.float().unsqueeze(-1)), torch.zeros((), device=scores.device))
    d = (p * (upstream_scores.float() - delta.float().unsqueeze(-1)) * scale).to(dtype) if want_grad else None
    return (p.to(dtype) if writes_probs else None), d
