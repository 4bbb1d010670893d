"""Gated short-convolution mixer (LFM2): the block that stands where attention would in a ``conv`` layer.

    b, c, x = split( in_proj(h) )                    three vectors of the hidden width per token
    y       = c * causal_depthwise_conv( b * x )     kernel of ``conv_kernel`` taps per channel (3 in the releases)
    out     = out_proj(y)

The convolution reads a token and the ``conv_kernel - 1`` tokens before it IN THE SAME DOCUMENT: in a packed row a tap
that would reach across a document's first token reads zero instead, which is what each document would see alone
(``ctx.positions`` marks the segments: a tap ``j`` back is live where the token's position is at least ``j``). The two
projections run on the framework's GEMM; the taps are a handful of shifted multiply-adds on ``[T, hidden]``.

While sampling, the cache keeps each sequence's last ``conv_kernel - 1`` products ``b * x`` per conv layer: prefill stores
them from the packed prompts, a decode step convolves them with the new token's product and shifts.

Whole rows only: a row cut over context-parallel or tensor-parallel ranks would cut the taps at the cut.
(The role of the reference's LFM2 entry in ``family_specs.py`` and of its segment markers for convolution mixers,
halo/models/segment_markers.py.)"""

from __future__ import annotations

import torch
from torch import nn

from halo_b200.ops import gemm


def segment_causal_conv(bx: torch.Tensor, kernel: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """``bx [T, H]``, ``kernel [H, L]`` (tap ``L - 1`` multiplies the token itself, tap ``L - 1 - j`` the token ``j``
    back), ``positions [T]`` (a token's index inside its document). Autograd through tensor ops."""
    L = kernel.shape[1]
    w = kernel.to(bx.dtype)
    out = bx * w[:, L - 1]
    for j in range(1, L):
        back = torch.nn.functional.pad(bx[:-j], (0, 0, j, 0)) if bx.shape[0] > j else torch.zeros_like(bx)
        live = (positions >= j).to(bx.dtype)[:, None]
        out = out + back * live * w[:, L - 1 - j]
    return out


class ShortConv(nn.Module):
    def __init__(self, cfg, dtype, device, tp_size: int = 1, layer_idx: int = 0):
        super().__init__()
        if tp_size > 1:
            raise ValueError("the short-convolution mixer is not cut over tensor-parallel ranks")
        self.cfg, self.layer_idx = cfg, layer_idx
        H, L = cfg.hidden_size, cfg.conv_kernel
        self.conv_in_proj = nn.Parameter(torch.empty(3 * H, H, dtype=dtype, device=device))
        self.conv_taps = nn.Parameter(torch.empty(H, 1, L, dtype=dtype, device=device))      # the hub's Conv1d shape
        self.conv_out_proj = nn.Parameter(torch.empty(H, H, dtype=dtype, device=device))
        self.window, self.sinks, self.lora, self.lowp = 0, None, None, ""

    def forward(self, h, ctx):
        if ctx.cp is not None or ctx.tp is not None:
            raise NotImplementedError("the short-convolution mixer runs on unsliced rows")
        H, L = self.cfg.hidden_size, self.cfg.conv_kernel
        bcx = gemm.linear(h, self.conv_in_proj)
        bx = bcx[:, :H] * bcx[:, 2 * H:]
        c = bcx[:, H:2 * H]
        kernel = self.conv_taps[:, 0, :]
        cache = ctx.kv_cache
        if cache is not None and cache.mode != "prefill":
            state = cache.conv_state(self.layer_idx, L - 1, bx)                 # [B, L-1, H]: oldest first
            taps = torch.cat([state, bx[:, None, :]], dim=1)                    # [B, L, H]
            conv = (taps * kernel.to(bx.dtype).t()[None]).sum(dim=1)
            state.copy_(taps[:, 1:])
        else:
            conv = segment_causal_conv(bx, kernel, ctx.positions)
            if cache is not None:
                cache.store_conv_tail(self.layer_idx, L - 1, bx)
        return gemm.linear((c * conv).contiguous(), self.conv_out_proj)
