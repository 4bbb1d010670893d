"""RMSNorm with the residual add folded in, forward and backward.

``rms_norm(x, w, eps)`` returns ``w * bf16(x * rstd)``; ``add_rms_norm(x, res, w, eps)`` returns
``(norm(x + res), x + res)`` from one pass over the row. CPU tensors take the PyTorch path with the
same rounding order, which is the oracle of the GPU tests.

Stands where the reference swaps in Liger's RMSNorm on dense Qwen3 and uses ATen's fused
``F.rms_norm`` on Qwen3-MoE (halo/model_loading/liger/family_specs.py:34-36,
halo/model_loading/liger/fused_modules.py:120-123).
"""

from __future__ import annotations

import torch

from . import _lib


def rms_norm_reference(x, weight, eps, residual=None):
    h = x if residual is None else (x + residual)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    y = weight * (hf * rstd).to(h.dtype)
    return (y, h) if residual is not None else y


def _supported(H: int) -> bool:
    return bool(_lib.lib().halo_rmsnorm_supported(_lib.c_int(H)))


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H).contiguous()
        r2 = residual.reshape(-1, H).contiguous() if residual is not None else None
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if r2 is not None else x2
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        L = _lib.lib()
        rc = L.halo_rmsnorm_fwd(
            _lib.ptr(x2), _lib.ptr(r2), _lib.ptr(weight), _lib.ptr(y), _lib.ptr(h if r2 is not None else None),
            _lib.ptr(rstd), _lib.c_ll(rows), _lib.c_int(H), _lib.c_float(eps), _lib.stream_ptr(x.device),
        )
        _lib.check(rc, "halo_rmsnorm_fwd")
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_res = r2 is not None
        ctx.shape = shape
        if r2 is not None:
            return y.reshape(shape), h.reshape(shape)
        return y.reshape(shape), None

    @staticmethod
    def backward(ctx, gy, gh):
        h, weight, rstd = ctx.saved_tensors
        rows, H = h.shape
        gy2 = gy.reshape(rows, H).contiguous()
        gh2 = gh.reshape(rows, H).contiguous() if (ctx.has_res and gh is not None) else None
        dx = torch.empty_like(h)
        L = _lib.lib()
        blocks = L.halo_rmsnorm_bwd_blocks(_lib.c_ll(rows), _lib.c_int(H))
        partial = torch.empty((max(blocks, 1), H), dtype=torch.float32, device=h.device)
        dw = torch.empty(H, dtype=torch.float32, device=h.device)
        rc = L.halo_rmsnorm_bwd(
            _lib.ptr(gy2), _lib.ptr(h), _lib.ptr(weight), _lib.ptr(rstd), _lib.ptr(gh2), _lib.ptr(dx),
            _lib.ptr(partial), _lib.ptr(dw), _lib.c_void_p(0), _lib.c_int(0), _lib.c_ll(rows), _lib.c_int(H),
            _lib.stream_ptr(h.device),
        )
        _lib.check(rc, "halo_rmsnorm_bwd")
        dx = dx.reshape(ctx.shape)
        return dx, (dx if ctx.has_res else None), dw.to(weight.dtype), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if not x.is_cuda or x.dtype != torch.bfloat16 or not _supported(x.shape[-1]):
        return rms_norm_reference(x, weight, eps)
    return _RMSNorm.apply(x, None, weight, eps)[0]


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Returns ``(rms_norm(x + residual), x + residual)``."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or not _supported(x.shape[-1]):
        return rms_norm_reference(x, weight, eps, residual)
    return _RMSNorm.apply(x, residual, weight, eps)
