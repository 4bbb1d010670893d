"""SwiGLU on a packed ``[rows, 2F]`` pre-activation (gate | up) as its own op, for the paths where the activation
cannot ride in a GEMM epilogue (an adapter's low-rank term is added to the pre-activation first).

CUDA bf16 tensors take the elementwise kernels (one pass each way, fp32 math); everything else takes the PyTorch
expression, which is also the oracle of the GPU test. The reference's counterpart is its GLU kernel pair
(halo/kernels/fused_glu.py:118-205).
"""

from __future__ import annotations

import torch

from . import _lib


def swiglu_reference(pre: torch.Tensor) -> torch.Tensor:
    F = pre.shape[-1] // 2
    g, u = pre[..., :F].float(), pre[..., F:].float()
    return (torch.nn.functional.silu(g) * u).to(pre.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pre):
        pre = pre.contiguous()
        rows, F2 = pre.shape
        act = torch.empty((rows, F2 // 2), dtype=pre.dtype, device=pre.device)
        if rows:
            rc = _lib.lib().halo_swiglu_fwd(_lib.ptr(pre), _lib.ptr(act), _lib.c_ll(rows), _lib.c_int(F2 // 2),
                                            _lib.stream_ptr(pre.device))
            _lib.check(rc, "halo_swiglu_fwd")
        ctx.save_for_backward(pre)
        return act

    @staticmethod
    def backward(ctx, dact):
        (pre,) = ctx.saved_tensors
        rows, F2 = pre.shape
        dpre = torch.empty_like(pre)
        if rows:
            rc = _lib.lib().halo_swiglu_bwd(_lib.ptr(pre), _lib.ptr(dact.contiguous()), _lib.ptr(dpre), _lib.c_ll(rows),
                                            _lib.c_int(F2 // 2), _lib.stream_ptr(pre.device))
            _lib.check(rc, "halo_swiglu_bwd")
        return dpre


def swiglu(pre: torch.Tensor) -> torch.Tensor:
    """``silu(pre[:, :F]) * pre[:, F:]`` for a 2-D ``pre``."""
    if pre.is_cuda and pre.dtype == torch.bfloat16 and pre.dim() == 2 and (pre.shape[1] // 2) % 8 == 0:
        return _SwiGLU.apply(pre)
    return swiglu_reference(pre)
