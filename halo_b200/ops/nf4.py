"""4-bit block quantisation of frozen base weights (QLoRA): every block of 64 values is divided by its absolute
maximum and each value is stored as the index of the nearest of 16 levels - ``nf4``: the quantiles of a standard
normal, normalised to [-1, 1] with an exact zero (Dettmers et al., 2023, appendix E); ``fp4``: the e2m1 grid
``+-{0, 0.5, 1, 1.5, 2, 3, 4, 6} / 6``. Two codes share a byte (first value in the high nibble). With ``nested``
the fp32 block maxima are themselves stored as 8-bit codes, evenly spaced in the logarithm between the smallest and
the largest maximum of each group of 256 blocks (relative error below 1.4 % even when a group spans three decades),
which brings the overhead from 0.5 to about 0.129 bits per value.

Dequantisation is a table lookup and one multiply (``csrc/nf4.cu`` for bf16 on CUDA, tensor operations elsewhere);
it runs once per layer and pass, just before the layer reads its weights. (The role of the bitsandbytes 4-bit storage the reference loads through
``load_in_4bit`` / ``use_bnb_nested_quant``, halo/model_loading/dtype.py:114-119.)"""

from __future__ import annotations

from dataclasses import dataclass

import torch

BLOCK = 64
NESTED_BLOCK = 256
NF4_LEVELS = (-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
              -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
              0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0)
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
FP4_LEVELS = tuple(-v / 6.0 for v in reversed(_E2M1)) + tuple(v / 6.0 for v in _E2M1)      # both signs of zero keep their code
KINDS = {"nf4": NF4_LEVELS, "fp4": FP4_LEVELS}
INT8 = "int8"          # 8-bit storage (``load_in_8bit``): one signed byte per value, code / 127 of the block maximum


def levels(kind: str, device=None) -> torch.Tensor:
    if kind not in KINDS:
        raise ValueError(f"4-bit format {kind!r}: choose from {', '.join(KINDS)}")
    return torch.tensor(KINDS[kind], dtype=torch.float32, device=device)


@dataclass
class Packed4bit:
    codes: torch.Tensor               # uint8 [n / 2] (two 4-bit codes per byte), or [n] signed bytes viewed as uint8 for int8
    absmax: torch.Tensor | None       # fp32 [n / BLOCK], or None when nested
    shape: tuple
    dtype: torch.dtype
    kind: str = "nf4"
    block: int = BLOCK
    nested_codes: torch.Tensor | None = None     # uint8 [n / BLOCK]: the maxima as 8-bit codes
    nested_scale: torch.Tensor | None = None     # fp32 [ceil(n / BLOCK / NESTED_BLOCK), 2]: log of the group's smallest and largest maximum

    @property
    def nbytes(self) -> int:
        parts = [self.codes, self.absmax, self.nested_codes, self.nested_scale]
        return sum(t.numel() * t.element_size() for t in parts if t is not None)

    def to(self, device) -> "Packed4bit":
        def move(t):
            return None if t is None else t.to(device)

        return Packed4bit(move(self.codes), move(self.absmax), self.shape, self.dtype, self.kind, self.block,
                          move(self.nested_codes), move(self.nested_scale))

    def block_maxima(self) -> torch.Tensor:
        if self.absmax is not None:
            return self.absmax
        n = self.nested_codes.numel()
        pad = (-n) % NESTED_BLOCK
        c = torch.nn.functional.pad(self.nested_codes.float(), (0, pad)).reshape(-1, NESTED_BLOCK) / 255.0
        lo, hi = self.nested_scale[:, :1], self.nested_scale[:, 1:]
        return torch.exp(lo + c * (hi - lo)).reshape(-1)[:n]


@torch.no_grad()
def quantize_4bit(w: torch.Tensor, kind: str = "nf4", nested: bool = False, block: int = BLOCK) -> Packed4bit:
    n = w.numel()
    if n % block or block % 2:
        raise ValueError(f"a tensor of {n} values does not split into blocks of {block}")
    x = w.detach().reshape(-1, block).float()
    absmax = x.abs().amax(dim=1)
    unit = x / absmax.clamp_min(1e-30)[:, None]
    if kind == INT8:
        if nested:
            raise ValueError("nested maxima are a 4-bit option")
        codes = torch.round(unit * 127.0).to(torch.int8).reshape(-1)
        return Packed4bit(codes.view(torch.uint8), absmax, tuple(w.shape), w.dtype, kind, block)
    table = levels(kind, w.device)
    # the nearest level: the table is sorted, so its index is the number of midpoints below the value
    codes = torch.bucketize(unit, (table[1:] + table[:-1]) / 2).to(torch.uint8).reshape(-1)
    packed = (codes[0::2] << 4) | codes[1::2]
    out = Packed4bit(packed, absmax, tuple(w.shape), w.dtype, kind, block)
    if nested:
        nb = absmax.numel()
        pad = (-nb) % NESTED_BLOCK
        groups = torch.nn.functional.pad(absmax, (0, pad)).reshape(-1, NESTED_BLOCK)
        top = groups.amax(dim=1, keepdim=True).clamp_min(1e-30)
        logs = torch.log(torch.where(groups > 0, groups, top))        # an all-zero block decodes to zero whatever its maximum
        lo, hi = logs.amin(dim=1, keepdim=True), logs.amax(dim=1, keepdim=True)
        q = torch.round((logs - lo) / (hi - lo).clamp_min(1e-12) * 255.0).clamp(0, 255)
        out.absmax, out.nested_codes = None, q.reshape(-1)[:nb].to(torch.uint8)
        out.nested_scale = torch.cat([lo, hi], dim=1)
    return out


def dequantize_4bit(p: Packed4bit, dtype: torch.dtype | None = None) -> torch.Tensor:
    dtype = dtype or p.dtype
    if p.kind == INT8:
        values = p.codes.view(torch.int8).reshape(-1, p.block).float() * (p.block_maxima() / 127.0)[:, None]
        return values.reshape(p.shape).to(dtype)
    if p.codes.is_cuda and dtype == torch.bfloat16 and p.block == BLOCK:
        # the sm_100a kernel (csrc/nf4.cu): 0.5 byte read and 2 bytes written per value, the same single rounding
        import ctypes

        from halo_b200.ops import _lib

        out = torch.empty(p.shape, dtype=torch.bfloat16, device=p.codes.device)
        maxima = p.block_maxima().float().contiguous()
        table = (ctypes.c_float * 16)(*KINDS[p.kind])
        rc = _lib.lib().halo_dequant_4bit_bf16(_lib.ptr(p.codes), _lib.ptr(maxima), _lib.ptr(out), _lib.c_ll(out.numel()), table,
                                               _lib.stream_ptr(out.device))
        _lib.check(rc, "halo_dequant_4bit_bf16")
        return out
    return dequantize_4bit_reference(p, dtype)


def dequantize_4bit_reference(p: Packed4bit, dtype: torch.dtype | None = None) -> torch.Tensor:
    """The tensor-op statement (every device): a table lookup and one multiply in fp32, one rounding."""
    table = levels(p.kind, p.codes.device)
    codes = torch.stack([p.codes >> 4, p.codes & 0xF], dim=1).reshape(-1, p.block).long()
    values = table[codes] * p.block_maxima()[:, None]
    return values.reshape(p.shape).to(dtype or p.dtype)


def quantization_error_bound(kind: str) -> float:
    """Largest distance from a value in [-1, 1] to its nearest level: the per-block relative error bound."""
    if kind == INT8:
        return 0.5 / 127.0
    t = levels(kind)
    return float((t[1:] - t[:-1]).max()) / 2
