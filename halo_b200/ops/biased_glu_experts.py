"""Routed experts with per-expert bias vectors and the clamped GLU of the gpt-oss family, as tensor operations.

``gate_up [E, 2F, H]`` holds the gate rows, then the up rows (the run-time bank layout; the hub stores them
interleaved column-wise and transposed). One expert computes

    pre  = x @ gate_up[e].T + gate_up_bias[e]
    gate = min(pre[:F], limit);  up = clamp(pre[F:], -limit, limit)
    y    = ((up + 1) * gate * sigmoid(alpha * gate)) @ down[e].T + down_bias[e]

and a token's output is the routing-weighted sum of its experts' ``y`` (the bias of the down projection is weighted
too). Tokens are sorted by expert once and each expert runs one pair of library GEMMs on its slice; autograd
differentiates it. This is the family's reference path: it reads the per-expert counts on the host, so it is not
capturable in a CUDA graph and does not dispatch over expert-parallel ranks.
(The role of the gpt-oss branch of halo/models/moe/experts.py and its ``gptoss`` activation.)"""

from __future__ import annotations

import torch

GLU_ALPHA = 1.702


def clamped_glu(pre: torch.Tensor, limit: float, alpha: float = GLU_ALPHA) -> torch.Tensor:
    """``pre [..., 2F]`` (gate half, then up half) -> ``[..., F]``."""
    gate, up = pre.chunk(2, dim=-1)
    gate = gate.clamp(max=limit)
    up = up.clamp(min=-limit, max=limit)
    return (up + 1) * (gate * torch.sigmoid(gate * alpha))


def biased_glu_experts(x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, gate_up: torch.Tensor, gate_up_bias: torch.Tensor,
                       down: torch.Tensor, down_bias: torch.Tensor, limit: float = 7.0, alpha: float = GLU_ALPHA) -> torch.Tensor:
    """``x [T, H]``, ``idx`` / ``w [T, k]`` (expert ids and routing weights) -> ``[T, H]``."""
    T, k = idx.shape
    E = gate_up.shape[0]
    flat = idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E).tolist()          # host read: the slices of the sorted rows
    token = order // k
    rows = x[token]
    weight = w.reshape(-1)[order].to(x.dtype)
    out = torch.zeros_like(x)
    start = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        sl = slice(start, start + n)
        pre = rows[sl] @ gate_up[e].t() + gate_up_bias[e]
        y = clamped_glu(pre, limit, alpha) @ down[e].t() + down_bias[e]
        out = out.index_add(0, token[sl], y * weight[sl, None])
        start += n
    return out


def biased_glu_experts_reference(x, idx, w, gate_up, gate_up_bias, down, down_bias, limit: float = 7.0, alpha: float = GLU_ALPHA,
                                 stored_dtype=None):
    """Every expert on every token, masked by the routing weights (dense form, fp32). ``stored_dtype``: the
    pre-activations are rounded to this dtype where the grouped kernels store them (product + bias, once),
    so that the clamps cut - and pass gradients - at the same elements as in the kernels: a value within one rounding
    step of ``limit`` is clamped in one form and not in the other otherwise."""
    E = gate_up.shape[0]
    xf = x.float()
    dense_w = torch.zeros(x.shape[0], E, dtype=torch.float32, device=x.device).scatter_add(1, idx.long(), w.float())
    pre = torch.einsum("th,efh->tef", xf, gate_up.float())
    pre = pre + gate_up_bias.float()[None]
    if stored_dtype is not None:
        pre = pre.to(stored_dtype).float()            # the grouped product's epilogue rounds accumulator + bias once
    y = torch.einsum("tef,ehf->teh", clamped_glu(pre, limit, alpha), down.float()) + down_bias.float()[None]
    return (y * dense_w[..., None]).sum(1).to(x.dtype)
