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
    def forward(ctx, layer, fwd_ctx, x, hooks, index):
        ctx.layer, ctx.fwd_ctx, ctx.hooks, ctx.index = layer, fwd_ctx, hooks, index
        ctx.save_for_backward(x)
        if hooks is not None:
            hooks.before_layer(index, backward=False)
        try:
            with torch.no_grad():
                return layer(x, fwd_ctx)
        finally:
            if hooks is not None:
                hooks.after_layer(index, backward=False)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        xin = x.detach().requires_grad_(True)
        hooks = ctx.hooks
        if hooks is not None:
            hooks.before_layer(ctx.index, backward=True)
        # the value of this second pass is never read (only its graph is): the layer's last op may skip
        # producing it
        ctx.fwd_ctx.output_unused = True
        try:
            with torch.enable_grad():
                out = ctx.layer(xin, ctx.fwd_ctx)
        finally:
            ctx.fwd_ctx.output_unused = False
        torch.autograd.backward(out, grad_out)
        if hooks is not None:
            hooks.after_layer(ctx.index, backward=True)
        return None, None, xin.grad, None, None


def recompute(layer, x: torch.Tensor, fwd_ctx, hooks=None, index: int = -1) -> torch.Tensor:
    """``hooks``: an object with ``before_layer(index, backward)`` / ``after_layer(index, backward)`` called around the
    layer's first pass and around its re-run + backward: the two windows in which the layer's parameters are needed
    (sharded parameters are gathered for exactly those windows, their gradients reduced right after the second)."""
    if not x.requires_grad:
        # nothing upstream needs a gradient, but the layer's parameters do: give autograd an edge
        x = x.detach().requires_grad_(True)
    return _Recompute.apply(layer, fwd_ctx, x, hooks, index)


class _OpenWindow(torch.autograd.Function):
    """Marks where a layer's parameter window opens in the forward and - in the backward, which reaches this node last
    of the layer's nodes - where it closes."""

    @staticmethod
    def forward(ctx, x, hooks, index):
        ctx.hooks, ctx.index = hooks, index
        hooks.before_layer(index, backward=False)
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        ctx.hooks.after_layer(ctx.index, backward=True)
        return grad, None, None


class _TailHooks:
    """The hooks of a layer's SECOND half when its first half runs with a graph of its own: the forward window was
    opened in front of the first half (so only its close remains here), and the backward window opens here, at the
    re-run of the second half, and stays open for the first half's backward (closed by :class:`_OpenWindow`)."""

    def __init__(self, hooks, index):
        self.hooks, self.index = hooks, index

    def before_layer(self, _index, backward):
        if backward:
            self.hooks.before_layer(self.index, backward=True)

    def after_layer(self, _index, backward):
        if not backward:
            self.hooks.after_layer(self.index, backward=False)


def recompute_second_half(first_half, second_half, x: torch.Tensor, fwd_ctx, hooks=None, index: int = -1) -> torch.Tensor:
    """The lighter policy: ``first_half`` (attention) keeps its graph, ``second_half`` (the feed-forward block) is re-run
    in the backward. With ``hooks`` the layer's parameters are needed in two windows: first pass of both halves; re-run and
    backward of the second half followed by the backward of the first. Parameters that the first half saved for its
    backward are leaf tensors whose storage is bound again when the second window opens, so the saved references read
    the gathered values of THAT window."""
    if hooks is None:
        return recompute(second_half, first_half(x, fwd_ctx), fwd_ctx)
    if not x.requires_grad:
        x = x.detach().requires_grad_(True)
    x = _OpenWindow.apply(x, hooks, index)
    return recompute(second_half, first_half(x, fwd_ctx), fwd_ctx, _TailHooks(hooks, index), index)
