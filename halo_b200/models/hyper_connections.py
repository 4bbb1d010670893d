"""Manifold-constrained hyper-connections: ``N`` residual streams per token instead of one.

Before each block a :class:`HyperConnection` reads the streams ``[T, N, H]`` and produces, per token, the weights
that *collapse* them into the block's input, the weights ``post`` that spread the block's output over the streams,
and a mixing matrix ``comb`` for the old streams, projected onto (nearly) doubly-stochastic matrices by
Sinkhorn-Knopp so the residual path neither amplifies nor loses signal. The head collapses the streams once more.
All per-token weights come from one skinny projection of the RMS-scaled flattened streams
(:func:`halo_b200.ops.streams.project_streams`), with fp32 parameters.

With the projection ``fn`` at zero and the biases at their initial values the collapse is the mean of the streams,
``post`` is one and ``comb`` is close to the identity: a freshly initialised hyper-connected model computes what
the plain residual model computes, and training moves away from there.

The forward follows the reference's fused form of the DeepSeek-V4 / GLM-5-Next modules
(halo/models/hyper_connections.py:26-101).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from halo_b200.ops.streams import collapse_streams, mix_streams, project_streams, sinkhorn_knopp

_IDENTITY_LOGIT = 8.0      # diagonal of the mixing logits at initialisation: softmax rows are one-hot to ~3e-4


class HyperConnection(nn.Module):
    def __init__(self, hidden: int, n_streams: int, sinkhorn_iters: int, eps: float, norm_eps: float, device=None):
        super().__init__()
        n = n_streams
        self.n, self.iters, self.eps, self.norm_eps = n, sinkhorn_iters, eps, norm_eps
        self.fn = nn.Parameter(torch.zeros(2 * n + n * n, n * hidden, dtype=torch.float32, device=device))
        self.base = nn.Parameter(torch.zeros(2 * n + n * n, dtype=torch.float32, device=device))
        self.scale = nn.Parameter(torch.ones(3, dtype=torch.float32, device=device))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        n = self.n
        self.fn.zero_()
        self.scale.fill_(1.0)
        self.base.zero_()
        self.base[:n].fill_(math.log(1.0 / n / (1.0 - 1.0 / n)) if n > 1 else 30.0)     # sigmoid -> 1 / n
        self.base[2 * n:].copy_((_IDENTITY_LOGIT * torch.eye(n)).reshape(-1))

    def forward(self, streams: torch.Tensor):
        """``streams [T, N, H]`` -> ``(post [T, N], comb [T, N, N], collapsed [T, H])``."""
        n = self.n
        projected = project_streams(streams, self.fn, self.norm_eps)
        pre_w, post_w, comb_w = projected.split([n, n, n * n], dim=-1)
        pre_b, post_b, comb_b = self.base.split([n, n, n * n])
        pre_scale, post_scale, comb_scale = self.scale.unbind(0)
        pre = torch.sigmoid(pre_w * pre_scale + pre_b) + self.eps
        post = 2.0 * torch.sigmoid(post_w * post_scale + post_b)
        comb_logits = comb_w.view(*comb_w.shape[:-1], n, n) * comb_scale + comb_b.view(n, n)
        comb = torch.softmax(comb_logits, dim=-1) + self.eps
        return post, sinkhorn_knopp(comb, self.iters, self.eps), collapse_streams(streams, pre)


def mixed(block: torch.Tensor, streams: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """The block's output spread over the streams plus the old streams mixed; both weights are rounded to the
    streams' dtype first, as the eager form of the families does."""
    return mix_streams(block, streams, post.to(streams.dtype), comb.to(streams.dtype))


class HyperHead(nn.Module):
    """Collapses the streams in front of the final norm with one sigmoid weight per stream."""

    def __init__(self, hidden: int, n_streams: int, eps: float, norm_eps: float, device=None):
        super().__init__()
        self.n, self.eps, self.norm_eps = n_streams, eps, norm_eps
        self.hc_fn = nn.Parameter(torch.zeros(n_streams, n_streams * hidden, dtype=torch.float32, device=device))
        self.hc_base = nn.Parameter(torch.zeros(n_streams, dtype=torch.float32, device=device))
        self.hc_scale = nn.Parameter(torch.ones(1, dtype=torch.float32, device=device))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self) -> None:
        n = self.n
        self.hc_fn.zero_()
        self.hc_scale.fill_(1.0)
        self.hc_base.fill_(math.log(1.0 / n / (1.0 - 1.0 / n)) if n > 1 else 30.0)

    def forward(self, streams: torch.Tensor) -> torch.Tensor:
        mixes = project_streams(streams, self.hc_fn, self.norm_eps)
        return collapse_streams(streams, torch.sigmoid(mixes * self.hc_scale + self.hc_base) + self.eps)


class GatedResidual(nn.Module):
    """The gated variant: the streams ``[T, N * H]`` are RMS-normalised per stream (``1 + w`` scaling), a low-rank
    gate (``down`` to ``rank`` features, SiLU, ``up`` back to ``N * H``, sigmoid) weights them and their mean over
    streams is the block's input; the block's output is injected into every stream with per-token gates
    ``2 * sigmoid(.)``. Follows the fused form of the reference's Flash-Next module
    (halo/models/families/qwen4_exp/gated_residual.py:99-112, 128-144)."""

    def __init__(self, hidden: int, n_streams: int, rank: int, norm_eps: float, dtype, device=None, seed: int = 0):
        super().__init__()
        self.n, self.eps = n_streams, norm_eps
        width = n_streams * hidden
        g = torch.Generator().manual_seed(seed)
        self.norm_weight = nn.Parameter(torch.zeros(width, dtype=torch.float32, device=device))

        def weight(rows, cols):
            return nn.Parameter((torch.randn(rows, cols, generator=g) * 0.02).to(dtype=dtype, device=device))

        self.mix_down, self.mix_up, self.inject = weight(rank, width), weight(width, rank), weight(n_streams, width)

    def forward(self, streams: torch.Tensor):
        """``streams [T, N, H]`` -> ``(block input [T, H], inject gates [T, N])``."""
        from halo_b200.ops.streams import gate_mix, grouped_rms_norm

        T, N, H = streams.shape
        normed = grouped_rms_norm(streams.reshape(T, N * H), self.norm_weight, self.eps, N)
        down = torch.nn.functional.linear(normed, self.mix_down)
        mixed = gate_mix(normed, down, self.mix_up, N)
        gates = 2.0 * torch.sigmoid(torch.nn.functional.linear(normed, self.inject) / N)
        return mixed, gates
