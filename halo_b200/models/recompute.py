"""Per-layer activation recomputation.

``recompute(layer, x, ctx)`` runs ``layer(x, ctx)`` without building a graph and keeps only ``x``;
in the backward pass the layer is run again with gradients enabled and differentiated on the spot,
so at any moment only one layer's intermediates are alive. Parameters receive their gradients
directly from the inner backward. The first (graph-free) pass tells the fused ops that nothing
needs to be saved, so they skip the extra outputs a differentiable forward writes.

Plays the part of the reference's gradient-checkpointing policy (full per-layer recompute,
halo/models/gradient_checkpointing.py:31-110), without a frame cache: routing is recomputed from
the same inputs and is deterministic.
"""

from __future__ import annotations

import torch


class _Recompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, layer, fwd_ctx, x):
        ctx.layer, ctx.fwd_ctx = layer, fwd_ctx
        ctx.save_for_backward(x)
        with torch.no_grad():
            return layer(x, fwd_ctx)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        xin = x.detach().requires_grad_(True)
        # the value of this second pass is never read (only its graph is): the layer's last op may skip
        # producing it
        ctx.fwd_ctx.output_unused = True
        try:
            with torch.enable_grad():
                out = ctx.layer(xin, ctx.fwd_ctx)
        finally:
            ctx.fwd_ctx.output_unused = False
        torch.autograd.backward(out, grad_out)
        return None, None, xin.grad


def recompute(layer, x: torch.Tensor, fwd_ctx) -> torch.Tensor:
    if not x.requires_grad:
        # nothing upstream needs a gradient, but the layer's parameters do: give autograd an edge
        x = x.detach().requires_grad_(True)
    return _Recompute.apply(layer, fwd_ctx, x)
