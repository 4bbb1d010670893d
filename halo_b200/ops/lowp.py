"""Block-scaled low precision: the OCP MX formats (``mxfp8``, ``mxfp4``: elements plus one power-of-two ``e8m0`` scale
per 32 elements of the contraction axis) and ``nvfp4`` (``e2m1`` elements, one ``e4m3`` scale per 16 elements, one fp32
power-of-two scale per tensor).

* :func:`quantize` / :func:`dequantize` - the stored form (:class:`BlockScaledTensor`: fp8 bytes or two e2m1 nibbles
  per byte, plus scales) for exporting weights;
* :func:`fake_quant` - the quantise-dequantise round trip in one pass, with a straight-through gradient, for
  quantisation-aware training; bf16 CUDA tensors run the sm_100a kernel (``csrc/lowp.cu``), everything else the
  tensor ops of :func:`fake_quant_reference`, which give the same bits;
* :class:`LowPrecisionLinear` semantics via :func:`lowp_linear`: both operands round-tripped along the contraction
  axis, the product itself on the bf16 tcgen05 GEMM (fp32 accumulation), so training sees the rounding the
  low-precision product will apply.

Exact arithmetic wherever the format allows it: exponents from ``frexp`` (no ``log2`` rounding at powers of two),
scaling by ``ldexp``, e2m1 rounding as a count of passed midpoints with ties to the even code.

Behavioural counterpart: halo/kernels/lowp/quantization.py:148-330, halo/kernels/lowp/linear.py.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

E4M3_MAX = 448.0
E2M1_MAX = 6.0
FORMATS = ("mxfp8", "mxfp4", "nvfp4")
BLOCK_SIZE = {"mxfp8": 32, "mxfp4": 32, "nvfp4": 16}
ELEMENT_MAX = {"mxfp8": E4M3_MAX, "mxfp4": E2M1_MAX, "nvfp4": E2M1_MAX}
_FMT_CODE = {"mxfp8": 0, "mxfp4": 1, "nvfp4": 2}
_E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_AMAX_FLOOR = torch.finfo(torch.float32).tiny
_E8M0_BIAS = 127


@dataclass(frozen=True)
class BlockScaledTensor:
    """``data``: ``float8_e4m3fn`` elements (mxfp8) or two e2m1 codes per ``uint8`` (low nibble first). ``scales``: one
    per block along the last axis - a biased ``uint8`` exponent for the MX formats, ``float8_e4m3fn`` for nvfp4, whose
    per-tensor ``global_scale`` multiplies on top."""

    data: torch.Tensor
    scales: torch.Tensor
    fmt: str
    global_scale: torch.Tensor | None = None


def _ceil_log2(r: torch.Tensor) -> torch.Tensor:
    """Smallest integer ``e`` with ``r <= 2**e`` for positive fp32 ``r``, exactly."""
    m, x = torch.frexp(r)
    return torch.where(m == 0.5, x - 1, x)


def _blocks(t: torch.Tensor, fmt: str) -> torch.Tensor:
    bs = BLOCK_SIZE[fmt]
    if t.shape[-1] % bs:
        raise ValueError(f"last axis of {t.shape[-1]} elements is not a multiple of {fmt}'s block of {bs}")
    return t.float().reshape(*t.shape[:-1], t.shape[-1] // bs, bs)


def _e2m1_codes(scaled: torch.Tensor) -> torch.Tensor:
    mag = scaled.abs().clamp(max=E2M1_MAX)
    code = ((mag > 0.25).to(torch.uint8) + (mag >= 0.75) + (mag > 1.25) + (mag >= 1.75) + (mag > 2.5) + (mag >= 3.5) + (mag > 5.0))
    return code.to(torch.uint8) | ((scaled < 0) | ((scaled == 0) & torch.signbit(scaled))).to(torch.uint8) << 3


def _e2m1_values(codes: torch.Tensor) -> torch.Tensor:
    levels = torch.tensor(_E2M1_LEVELS, dtype=torch.float32, device=codes.device)
    mag = levels[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


def _mx_exponent(blocks: torch.Tensor, fmt: str) -> torch.Tensor:
    amax = blocks.abs().amax(-1, keepdim=True).clamp(min=_AMAX_FLOOR)
    return _ceil_log2(amax / ELEMENT_MAX[fmt]).clamp(-_E8M0_BIAS, _E8M0_BIAS).to(torch.int32)


def nvfp4_global_scale(amax: torch.Tensor) -> torch.Tensor:
    """The power of two that brings a tensor's ``amax`` to at most ``448 * 6``: the largest block scale then fits e4m3,
    and, being a power of two, it leaves e4m3 rounding unchanged, so any slice of the tensor quantises as the whole."""
    return torch.ldexp(torch.ones_like(amax, dtype=torch.float32), _ceil_log2(amax.float().clamp(min=_AMAX_FLOOR) / (E4M3_MAX * E2M1_MAX)))


def quantize(t: torch.Tensor, fmt: str, global_scale: torch.Tensor | None = None) -> BlockScaledTensor:
    """Quantise along the last axis."""
    if fmt not in FORMATS:
        raise ValueError(f"unknown format {fmt!r}; known: {FORMATS}")
    blocks = _blocks(t, fmt)
    if fmt == "nvfp4":
        gs = nvfp4_global_scale(blocks.abs().amax()) if global_scale is None else global_scale.float()
        amax = blocks.abs().amax(-1, keepdim=True)
        scale = (amax / E2M1_MAX / gs).clamp(max=E4M3_MAX).to(torch.float8_e4m3fn)
        unit = scale.float() * gs
        codes = _e2m1_codes(blocks / torch.where(unit == 0, torch.ones_like(unit), unit)).reshape(t.shape)
        return BlockScaledTensor(codes[..., 0::2] | (codes[..., 1::2] << 4), scale.squeeze(-1), fmt, gs)
    e = _mx_exponent(blocks, fmt)
    scaled = torch.ldexp(blocks, -e).clamp(-ELEMENT_MAX[fmt], ELEMENT_MAX[fmt])
    scales = (e + _E8M0_BIAS).to(torch.uint8).squeeze(-1)
    if fmt == "mxfp8":
        return BlockScaledTensor(scaled.to(torch.float8_e4m3fn).reshape(t.shape), scales, fmt)
    codes = _e2m1_codes(scaled).reshape(t.shape)
    return BlockScaledTensor(codes[..., 0::2] | (codes[..., 1::2] << 4), scales, fmt)


def dequantize(q: BlockScaledTensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    bs = BLOCK_SIZE[q.fmt]
    if q.fmt == "mxfp8":
        values = q.data.float()
    else:
        codes = torch.stack([q.data & 0xF, q.data >> 4], dim=-1).reshape(*q.data.shape[:-1], q.data.shape[-1] * 2)
        values = _e2m1_values(codes)
    blocks = values.reshape(*values.shape[:-1], values.shape[-1] // bs, bs)
    if q.fmt == "nvfp4":
        out = blocks * (q.scales.float() * q.global_scale).unsqueeze(-1)
    else:
        out = torch.ldexp(blocks, (q.scales.to(torch.int32) - _E8M0_BIAS).unsqueeze(-1))
    return out.reshape(values.shape).to(dtype)


def fake_quant_reference(t: torch.Tensor, fmt: str) -> torch.Tensor:
    """The round trip ``dequantize(quantize(t))`` in ``t``'s dtype, as tensor ops."""
    return dequantize(quantize(t, fmt), t.dtype)


class _FakeQuant(torch.autograd.Function):
    """Straight-through: the gradient passes unchanged (the rounding has zero gradient almost everywhere)."""

    @staticmethod
    def forward(ctx, t, fmt):
        return _fake_quant_forward(t, fmt)

    @staticmethod
    def backward(ctx, g):
        return g, None


def _fake_quant_forward(t: torch.Tensor, fmt: str) -> torch.Tensor:
    bs = BLOCK_SIZE[fmt]
    if t.shape[-1] % bs:
        raise ValueError(f"last axis of {t.shape[-1]} elements is not a multiple of {fmt}'s block of {bs}")
    if t.is_cuda and t.dtype == torch.bfloat16:
        x = t.contiguous()
        if x.data_ptr() % 16 == 0:
            y = torch.empty_like(x)
            amax = x.abs().amax().float().reshape(1) if fmt == "nvfp4" else None
            _lib.check(_lib.lib().halo_fake_quant_bf16(_lib.ptr(x), _lib.ptr(y), _lib.c_ll(x.numel()), _lib.c_int(_FMT_CODE[fmt]),
                                                       _lib.ptr(amax), _lib.stream_ptr(x.device)), "halo_fake_quant_bf16")
            return y
    return fake_quant_reference(t, fmt)


def fake_quant(t: torch.Tensor, fmt: str) -> torch.Tensor:
    """Quantise-dequantise along the last axis, straight-through gradient."""
    if fmt not in FORMATS:
        raise ValueError(f"unknown format {fmt!r}; known: {FORMATS}")
    if torch.is_grad_enabled() and t.requires_grad:
        return _FakeQuant.apply(t, fmt)
    return _fake_quant_forward(t, fmt)


def lowp_linear(x: torch.Tensor, weight: torch.Tensor, fmt: str, weight_fmt: str | None = None) -> torch.Tensor:
    """``x @ weight.T`` as the low-precision product would compute it: activations and weights both rounded to
    ``fmt`` (weights to ``weight_fmt`` when given) in blocks along the contraction axis, fp32 accumulation."""
    from .gemm import linear

    return linear(fake_quant(x, fmt), fake_quant(weight, weight_fmt or fmt))


class WeightRoundTripCache:
    """The rounded copy of a weight, rebuilt only when the weight changes (its ``_version`` counter moves with every
    in-place optimizer update): micro-batches of one step share one round trip."""

    def __init__(self):
        self._entries: dict[int, tuple[int, str, torch.Tensor]] = {}

    def get(self, weight: torch.Tensor, fmt: str) -> torch.Tensor:
        key = id(weight)
        hit = self._entries.get(key)
        if hit is not None and hit[0] == weight._version and hit[1] == fmt:
            return hit[2]
        with torch.no_grad():
            rounded = fake_quant(weight.detach(), fmt)
        self._entries[key] = (weight._version, fmt, rounded)
        return rounded

    def clear(self) -> None:
        self._entries.clear()


# the sixteen values of a 4-bit e2m1 code (sign, two exponent bits, one mantissa bit)
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def unpack_mxfp4_blocks(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """``blocks`` uint8 ``[..., G, B/2]`` (two e2m1 codes per byte, the low nibble first) and ``scales`` uint8
    ``[..., G]`` (a power-of-two exponent with bias 127 per block of B values) -> fp32 ``[..., G * B]``."""
    if blocks.dtype != torch.uint8 or scales.dtype != torch.uint8 or blocks.shape[:-1] != scales.shape:
        raise ValueError(f"packed blocks {tuple(blocks.shape)} {blocks.dtype} do not match scales {tuple(scales.shape)} {scales.dtype}")
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    lo, hi = lut[(blocks & 0x0F).long()], lut[(blocks >> 4).long()]
    vals = torch.stack([lo, hi], dim=-1).reshape(*blocks.shape[:-1], blocks.shape[-1] * 2)
    vals = torch.ldexp(vals, (scales.to(torch.int32) - 127)[..., None])
    return vals.reshape(*scales.shape[:-1], scales.shape[-1] * blocks.shape[-1] * 2)
