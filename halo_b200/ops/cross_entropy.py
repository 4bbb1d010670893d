"""Output head fused with its loss: the ``[T, V]`` logits plane is never materialised.

``fused_linear_cross_entropy`` walks the tokens in chunks. Per chunk: logits = h W^T on the
tcgen05 GEMM, one kernel turns the chunk into ``scale * (softmax - onehot)`` in place while
emitting the per-row loss, and two more GEMMs produce the chunk's dh and accumulate dW (fp32).
Gradients are therefore ready when the forward returns; the backward only hands them out.

``linear_logprobs`` is the scoring twin used by the RL trainers: per-token log-probability (and
entropy) of the labels, with a recompute backward.

Stands where the reference uses Liger's fused linear cross-entropy and its own chunked
hidden-state log-prob sweep (halo/kernels/head_logprobs.py:293, halo/kernels/logprobs.py:48-72).
"""

from __future__ import annotations

import torch

from . import _lib
from .gemm import matmul

IGNORE_INDEX = -100
DEFAULT_CHUNK_ROWS = 4096


def shift_labels_left(labels: torch.Tensor, ignore_index: int = IGNORE_INDEX) -> torch.Tensor:
    """Next-token targets: position t is scored against token t+1; the last position is ignored."""
    out = torch.full_like(labels, ignore_index)
    out[..., :-1] = labels[..., 1:]
    return out


def _ce_chunk_reference(logits, labels, ignore_index):
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    valid = labels != ignore_index
    safe = labels.clamp_min(0)
    tgt = lf.gather(-1, safe[:, None])[:, 0]
    loss = torch.where(valid, lse - tgt, torch.zeros_like(lse))
    return loss, lse


def _ce_inplace(logits, labels, grad_scale, row_scale, ignore_index):
    """In place: logits <- grad_scale * row_scale * (softmax - onehot); returns (loss_rows, lse)."""
    rows, V = logits.shape
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    rc = _lib.lib().halo_cross_entropy_inplace(
        _lib.ptr(logits), _lib.ptr(labels), _lib.ptr(grad_scale), _lib.ptr(row_scale), _lib.ptr(loss),
        _lib.ptr(lse), _lib.c_ll(rows), _lib.c_ll(logits.stride(0)), _lib.c_int(V), _lib.c_ll(ignore_index),
        _lib.stream_ptr(logits.device),
    )
    _lib.check(rc, "halo_cross_entropy_inplace")
    return loss, lse


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, grad_scale, chunk_rows, ignore_index):
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        need_dh = hidden.requires_grad
        need_dw = weight.requires_grad
        dh = torch.empty_like(hidden) if need_dh else None
        dw32 = torch.zeros((V, H), dtype=torch.float32, device=dev) if need_dw else None
        loss_sum = torch.zeros((), dtype=torch.float32, device=dev)
        Vp = (V + 7) // 8 * 8
        buf = torch.empty((min(chunk_rows, max(T, 1)), Vp), dtype=torch.bfloat16, device=dev)
        for s in range(0, T, chunk_rows):
            e = min(T, s + chunk_rows)
            hc = hidden[s:e]
            logits = buf[: e - s, :V]
            matmul(hc, weight, out=logits)
            loss_rows, _ = _ce_inplace(logits, labels[s:e], grad_scale, None, ignore_index)
            loss_sum += loss_rows.sum()
            if need_dh:
                matmul(logits, weight, b_t=False, out=dh[s:e])
            if need_dw:
                matmul(logits, hc, a_t=True, b_t=False, out=dw32, accumulate=True)
        ctx.save_for_backward(dh, dw32.to(weight.dtype) if need_dw else None)
        return loss_sum * grad_scale


    @staticmethod
    def backward(ctx, g):
        dh, dw = ctx.saved_tensors
        # the stored gradients already carry grad_scale; g is the upstream scalar (1 for a plain loss)
        if dh is not None:
            dh = dh * g.to(dh.dtype)
        if dw is not None:
            dw = dw * g.to(dw.dtype)
        return dh, dw, None, None, None, None


def fused_linear_cross_entropy(
    hidden: torch.Tensor,
    weight: torch.Tensor,
    labels: torch.Tensor,
    normalizer: torch.Tensor | float | None = None,
    chunk_rows: int = DEFAULT_CHUNK_ROWS,
    ignore_index: int = IGNORE_INDEX,
) -> torch.Tensor:
    """Sum over tokens of CE(h W^T, label) divided by ``normalizer`` (default: number of scored tokens).

    ``labels`` are already shifted (see :func:`shift_labels_left`). ``normalizer`` may be a device
    scalar so that no host synchronisation is needed.
    """
    hidden = hidden.reshape(-1, hidden.shape[-1])
    labels = labels.reshape(-1)
    if normalizer is None:
        normalizer = (labels != ignore_index).sum().clamp_min(1).to(torch.float32)
    if not hidden.is_cuda:
        total = hidden.new_zeros((), dtype=torch.float32)
        for s in range(0, hidden.shape[0], chunk_rows):
            e = min(hidden.shape[0], s + chunk_rows)
            logits = (hidden[s:e] @ weight.t()).to(hidden.dtype)
            loss, _ = _ce_chunk_reference(logits, labels[s:e], ignore_index)
            total = total + loss.sum()
        return total / normalizer
    if not torch.is_tensor(normalizer):
        normalizer = torch.tensor(float(normalizer), dtype=torch.float32, device=hidden.device)
    grad_scale = (1.0 / normalizer.to(torch.float32)).reshape(1)
    return _FusedLinearCE.apply(hidden.contiguous(), weight, labels.contiguous(), grad_scale, chunk_rows, ignore_index)


class _LinearLogprobs(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, chunk_rows, ignore_index, want_entropy):
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        logp = torch.empty(T, dtype=torch.float32, device=dev)
        ent = torch.empty(T, dtype=torch.float32, device=dev) if want_entropy else None
        Vp = (V + 7) // 8 * 8
        buf = torch.empty((min(chunk_rows, max(T, 1)), Vp), dtype=torch.bfloat16, device=dev)
        L = _lib.lib()
        for s in range(0, T, chunk_rows):
            e = min(T, s + chunk_rows)
            logits = buf[: e - s, :V]
            matmul(hidden[s:e], weight, out=logits)
            rc = L.halo_logprob_entropy(
                _lib.ptr(logits), _lib.ptr(labels[s:e]), _lib.ptr(logp[s:e]),
                _lib.ptr(ent[s:e]) if want_entropy else _lib.c_void_p(0), _lib.c_ll(e - s),
                _lib.c_ll(logits.stride(0)), _lib.c_int(V), _lib.c_ll(ignore_index), _lib.stream_ptr(dev),
            )
            _lib.check(rc, "halo_logprob_entropy")
        ctx.save_for_backward(hidden, weight, labels)
        ctx.meta = (chunk_rows, ignore_index)
        ctx.mark_non_differentiable(*( [ent] if want_entropy else [] ))
        return (logp, ent) if want_entropy else (logp, None)

    @staticmethod
    def backward(ctx, g_logp, _g_ent):
        hidden, weight, labels = ctx.saved_tensors
        chunk_rows, ignore_index = ctx.meta
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        dh = torch.empty_like(hidden) if ctx.needs_input_grad[0] else None
        dw32 = torch.zeros((V, H), dtype=torch.float32, device=dev) if ctx.needs_input_grad[1] else None
        Vp = (V + 7) // 8 * 8
        buf = torch.empty((min(chunk_rows, max(T, 1)), Vp), dtype=torch.bfloat16, device=dev)
        neg = (-g_logp).to(torch.float32).contiguous()
        for s in range(0, T, chunk_rows):
            e = min(T, s + chunk_rows)
            logits = buf[: e - s, :V]
            matmul(hidden[s:e], weight, out=logits)
            # d logits = g * (onehot - softmax) = (-g) * (softmax - onehot)
            _ce_inplace(logits, labels[s:e], None, neg[s:e], ignore_index)
            if dh is not None:
                matmul(logits, weight, b_t=False, out=dh[s:e])
            if dw32 is not None:
                matmul(logits, hidden[s:e], a_t=True, b_t=False, out=dw32, accumulate=True)
        return dh, (dw32.to(weight.dtype) if dw32 is not None else None), None, None, None, None


def linear_logprobs(hidden, weight, labels, chunk_rows=DEFAULT_CHUNK_ROWS, ignore_index=IGNORE_INDEX,
                    want_entropy=False):
    """Per-token ``log p(label)`` (0 where ignored) and optionally the entropy of the distribution."""
    hidden = hidden.reshape(-1, hidden.shape[-1])
    labels = labels.reshape(-1)
    if not hidden.is_cuda:
        outs, ents = [], []
        for s in range(0, hidden.shape[0], chunk_rows):
            e = min(hidden.shape[0], s + chunk_rows)
            logits = (hidden[s:e] @ weight.t()).to(hidden.dtype)
            loss, lse = _ce_chunk_reference(logits, labels[s:e], ignore_index)
            outs.append(-loss)
            if want_entropy:
                lf = logits.float()
                p = torch.softmax(lf, dim=-1)
                ents.append(lse - (p * lf).sum(-1))
        logp = torch.cat(outs) if outs else hidden.new_zeros(0, dtype=torch.float32)
        return (logp, torch.cat(ents).detach()) if want_entropy else (logp, None)
    return _LinearLogprobs.apply(hidden.contiguous(), weight, labels.contiguous(), chunk_rows, ignore_index, want_entropy)
