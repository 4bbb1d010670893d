"""bf16 matrix products on the tcgen05 GEMM kernel, with the autograd wiring of a linear layer.

``matmul(a, b, a_t, b_t)`` computes ``op(a) @ op(b)`` where a transposed operand is read in place
through the kernel's MN-major operand mode, so the three products of a linear layer

    y = x W^T          (forward)
    dx = dy W          (data gradient)
    dW = dy^T x        (weight gradient)

never materialise a transpose. CPU tensors take the PyTorch path (fp32 accumulate, one rounding),
which is also the oracle the GPU tests compare against.

Stands where the reference calls cuBLAS through ``F.linear`` and ``mm_fp32``
(halo/kernels/fp32_matmul.py:1-55).
"""

from __future__ import annotations

import torch

from . import _lib

EPI_STORE_BF16 = 0
EPI_STORE_F32 = 1
EPI_ACCUM_BF16 = 2
EPI_ACCUM_F32 = 3
EPI_SWIGLU = 4

GEMM_ALIGNMENT = 8  # elements: every leading dimension must be a multiple of 16 bytes


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError("expected a 2-D tensor")
    if t.stride(1) != 1 or t.stride(0) % GEMM_ALIGNMENT or t.data_ptr() % 16:
        t = t.contiguous()
    if t.stride(0) % GEMM_ALIGNMENT:
        raise ValueError(f"leading dimension {t.stride(0)} is not a multiple of {GEMM_ALIGNMENT}")
    return t


def matmul(
    a: torch.Tensor,
    b: torch.Tensor,
    a_t: bool = False,
    b_t: bool = True,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    accumulate: bool = False,
    alpha: float = 1.0,
) -> torch.Tensor:
    """``out (+)= alpha * op(a) @ op(b)``.

    ``a_t``: ``a`` is stored ``[K, M]`` (else ``[M, K]``). ``b_t``: ``b`` is stored ``[N, K]``, the
    layout of an ``nn.Linear`` weight (else ``[K, N]``).
    """
    M, K = (a.shape[1], a.shape[0]) if a_t else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[0], b.shape[1]) if b_t else (b.shape[1], b.shape[0])
    if K != Kb:
        raise ValueError(f"reduction sizes differ: {K} vs {Kb}")
    if out is not None:
        out_dtype = out.dtype
    if out_dtype is None:
        # the kernel rounds its fp32 accumulators to bf16; the PyTorch path keeps the operands' precision, so an
        # fp32 model on the CPU really computes in fp32
        out_dtype = torch.bfloat16 if a.is_cuda else a.dtype
    if not a.is_cuda:
        af = a.float().t() if a_t else a.float()
        bf = b.float().t() if b_t else b.float()
        res = (af @ bf) * alpha
        if out is None:
            return res.to(out_dtype)
        if accumulate:
            out.copy_((out.float() + res).to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("the tcgen05 GEMM takes bf16 operands")
    a = _row_major_2d(a)
    b = _row_major_2d(b)
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out.stride(1) != 1 or tuple(out.shape) != (M, N):
        raise ValueError("output must be [M, N] with contiguous rows")
    if out_dtype == torch.bfloat16:
        epi = EPI_ACCUM_BF16 if accumulate else EPI_STORE_BF16
        if out.stride(0) % 8 or N % 8:
            raise ValueError("bf16 output needs N and its leading dimension to be multiples of 8")
    elif out_dtype == torch.float32:
        epi = EPI_ACCUM_F32 if accumulate else EPI_STORE_F32
        if out.stride(0) % 4 or N % 4:
            raise ValueError("fp32 output needs N and its leading dimension to be multiples of 4")
    else:
        raise TypeError(f"unsupported output dtype {out_dtype}")
    if M == 0 or N == 0:
        return out
    if K == 0:
        if not accumulate:
            out.zero_()
        return out
    L = _lib.lib()
    rc = L.halo_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.c_void_p(0),
        _lib.c_int(M), _lib.c_int(N), _lib.c_int(K),
        _lib.c_ll(a.stride(0)), _lib.c_ll(b.stride(0)), _lib.c_ll(out.stride(0)), _lib.c_ll(0),
        _lib.c_int(1 if a_t else 0), _lib.c_int(0 if b_t else 1), _lib.c_int(epi),
        _lib.c_float(alpha), _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr(a.device),
    )
    _lib.check(rc, "halo_gemm_bf16")
    return out


def swiglu_matmul(x: torch.Tensor, w_gate_up: torch.Tensor, save_pre: bool = False):
    """``act = silu(x Wg^T) * (x Wu^T)`` with ``w_gate_up = [Wg; Wu]`` stacked ``[2F, K]``.

    One GEMM; the activation is applied in the epilogue while the tile is still in registers.
    With ``save_pre`` the bf16 pre-activations ``[gate | up]`` are written too (for backward).
    """
    M, K = x.shape
    F2 = w_gate_up.shape[0]
    F = F2 // 2
    if not x.is_cuda:
        pre = (x.float() @ w_gate_up.float().t()).to(x.dtype)
        g, u = pre[:, :F].float(), pre[:, F:].float()
        act = (torch.nn.functional.silu(g) * u).to(x.dtype)
        return (act, pre) if save_pre else (act, None)
    x = _row_major_2d(x)
    w = _row_major_2d(w_gate_up)
    if F % 8:
        raise ValueError("SwiGLU width must be a multiple of 8")
    act = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    pre = torch.empty((M, F2), dtype=torch.bfloat16, device=x.device) if save_pre else None
    if M == 0:
        return act, pre
    L = _lib.lib()
    rc = L.halo_gemm_bf16(
        _lib.ptr(x), _lib.ptr(w), _lib.ptr(act), _lib.ptr(pre),
        _lib.c_int(M), _lib.c_int(F2), _lib.c_int(K),
        _lib.c_ll(x.stride(0)), _lib.c_ll(w.stride(0)), _lib.c_ll(F), _lib.c_ll(F2),
        _lib.c_int(0), _lib.c_int(0), _lib.c_int(EPI_SWIGLU),
        _lib.c_float(1.0), _lib.ptr(_lib.status_word(x.device)), _lib.stream_ptr(x.device),
    )
    _lib.check(rc, "halo_gemm_bf16(swiglu)")
    return act, pre


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        ctx.save_for_backward(x2, weight)
        ctx.in_shape = shape
        y = matmul(x2, weight, a_t=False, b_t=True)
        return y.reshape(*shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, weight = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if gy2.dtype != x2.dtype:
            gy2 = gy2.to(x2.dtype)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = matmul(gy2, weight, a_t=False, b_t=False).reshape(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            gw = matmul(gy2, x2, a_t=True, b_t=False)
        return gx, gw


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T`` with all three products on the tcgen05 kernel (no bias: the model families
    built here have none on their projections)."""
    return _Linear.apply(x, weight)
