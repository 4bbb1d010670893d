"""AdamW with bf16 parameters and bf16 moments (6 bytes of optimizer state per parameter).

Arithmetic is fp32; the weight and the second moment are written back with stochastic rounding,
the first moment with round-to-nearest. The rounding noise is a pure function of
``(key, step, blake2b(parameter name), element offset)``, so replicas round alike and a resumed
run rounds exactly as the uninterrupted one. On CUDA every bf16 parameter of a group is stepped by
one multi-tensor kernel launch; the global-norm clip coefficient and the non-finite skip flag are
read from device memory inside that kernel, so clipping costs no pass over the gradients and a
skipped step costs no host synchronisation. fp32 parameters (an fp32 router, say) take a plain
fp32 AdamW step with the same clip / skip contract.

The CPU implementation below is the bit-exact twin of the kernel and the oracle of its tests.

Counterpart of halo/optimizers/adamw_bf16.py:378-499 (optimizer), :99-187 (fused step),
halo/optimizers/stochastic_rounding.py:30-63 (noise keying), halo/optimizers/step_skip.py:15-55.
"""

from __future__ import annotations

import ctypes
import hashlib
import math
from typing import Iterable

import numpy as np
import torch

from halo_b200.ops import _lib

SR_KEY = 0xB165EED
_MASK64 = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK64
    return x ^ (x >> 31)


def param_name_hash(name: str) -> int:
    """Ranks may hold different parameter lists; hashing the name keeps a replicated parameter's
    noise identical everywhere."""
    return int.from_bytes(hashlib.blake2b(name.encode(), digest_size=8).digest(), "little")


def sr_key_pair(key: int, step: int, name_hash: int) -> tuple[int, int]:
    mixed = splitmix64(splitmix64((key ^ step) & _MASK64) ^ name_hash)
    return mixed & 0xFFFFFFFF, (mixed >> 32) & 0xFFFFFFFF


def philox4x32_10(k0: int, k1: int, counter: np.ndarray) -> np.ndarray:
    """Vectorised Philox-4x32-10. ``counter``: uint64 [n] (low / high words form c0 / c1; c2 = c3 = 0).
    Returns uint32 [n, 4]."""
    c0 = (counter & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    c1 = (counter >> np.uint64(32)).astype(np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = m0 * c0
        p1 = m1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        n0 = hi1 ^ c1 ^ np.uint64(k0)
        n2 = hi0 ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0 & mask, lo1, n2 & mask, lo0
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def _sr_to_bf16(x: torch.Tensor, noise16: torch.Tensor) -> torch.Tensor:
    bits = x.contiguous().view(torch.int32) + noise16.to(torch.int32)
    bits = bits & -65536
    return bits.view(torch.float32).to(torch.bfloat16)


def adamw_bf16_step_reference(p, g, m, v, *, beta1, beta2, step_size, bc2_sqrt, eps, wd_factor, key, step,
                              name_hash, grad_scale=None, skip=False):
    """Bit-exact CPU twin of the CUDA step for one tensor (updates p, m, v in place)."""
    if skip:
        return
    n = p.numel()
    f32 = lambda x: torch.tensor(x, dtype=torch.float32)  # noqa: E731
    gf = g.detach().reshape(-1).float()
    if grad_scale is not None:
        sc = torch.as_tensor(grad_scale, dtype=torch.float32)
        if g.dtype == torch.bfloat16:
            sc = sc.bfloat16().float()
            gf = (gf * sc).bfloat16().float()
        else:
            gf = gf * sc
    pf, mf, vf = (t.detach().reshape(-1).float() for t in (p, m, v))
    omb1 = f32(1.0 - float(np.float32(beta1)))
    omb2 = f32(1.0 - float(np.float32(beta2)))
    mn = mf * f32(beta1) + gf * omb1
    vn = vf * f32(beta2) + (gf * gf) * omb2
    denom = vn.sqrt() / f32(bc2_sqrt) + f32(eps)
    pn = pf * f32(wd_factor) - (f32(step_size) * mn) / denom
    k0, k1 = sr_key_pair(key, step, name_hash)
    quads = (n + 3) // 4
    rnd = philox4x32_10(k0, k1, np.arange(quads, dtype=np.uint64)).reshape(-1)[:n]
    rnd_t = torch.from_numpy(rnd.astype(np.int64))
    v_noise = (rnd_t >> 16) & 0xFFFF
    p_noise = rnd_t & 0xFFFF
    m.detach().reshape(-1).copy_(mn.bfloat16())
    v.detach().reshape(-1).copy_(_sr_to_bf16(vn, v_noise))
    p.detach().reshape(-1).copy_(_sr_to_bf16(pn, p_noise))


class _DeviceTable:
    """Pointer / size tables of one parameter group, rebuilt only when a pointer changes."""

    def __init__(self):
        self.sig = None
        self.tensors = None

    def build(self, params, grads, ms, vs, hashes, device):
        L = _lib.lib()
        epb = int(L.halo_adam_elems_per_block())
        sig = tuple((p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel())
                    for p, g, m, v in zip(params, grads, ms, vs))
        if sig == self.sig:
            return self.tensors
        n = len(params)
        arr = np.zeros((6, n), dtype=np.uint64)
        blocks = [0]
        for i, (p, g, m, v, h) in enumerate(zip(params, grads, ms, vs, hashes)):
            arr[0, i], arr[1, i], arr[2, i], arr[3, i] = p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr()
            arr[4, i] = p.numel()
            arr[5, i] = h
            blocks.append(blocks[-1] + (p.numel() + epb - 1) // epb)
        tab = torch.from_numpy(arr.view(np.int64)).to(device)
        bstart = torch.tensor(blocks, dtype=torch.int32).to(device)
        self.sig = sig
        self.tensors = (tab, bstart, blocks[-1])
        return self.tensors


class AdamWBF16(torch.optim.Optimizer):
    """``params``: ``(name, parameter)`` pairs or param-group dicts with ``params`` and ``param_names``."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 key: int = SR_KEY):
        if lr < 0.0 or eps < 0.0 or not 0.0 <= betas[0] < 1.0 or not 0.0 <= betas[1] < 1.0:
            raise ValueError("invalid AdamWBF16 hyper-parameters")
        params = list(params)
        if params and isinstance(params[0], tuple):
            names = [n for n, _ in params]
            params = [{"params": [p for _, p in params], "param_names": names}]
        super().__init__(params, {"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay})
        for group in self.param_groups:
            if "param_names" not in group or len(group["param_names"]) != len(group["params"]):
                raise ValueError(
                    "AdamWBF16 keys its stochastic rounding by parameter name: build it from (name, param) pairs "
                    "or groups carrying 'param_names'."
                )
        self.key = key
        self._grad_scale: torch.Tensor | None = None
        self._skip: torch.Tensor | None = None
        self._tables: dict[tuple[int, str], _DeviceTable] = {}

    # -- clip / skip hand-off -------------------------------------------------------------
    def defer_grad_scale(self, scale: torch.Tensor | None) -> None:
        """Multiply every gradient by ``scale`` (device fp32 scalar) inside the next step."""
        self._grad_scale = None if scale is None else scale.detach().to(torch.float32).reshape(1)

    def arm_skip(self, flag: torch.Tensor | None) -> None:
        """``flag``: device int32 scalar; a non-zero value turns the next step into a no-op."""
        self._skip = None if flag is None else flag.reshape(1)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._grad_scale = None
        super().zero_grad(set_to_none=set_to_none)

    # -- state ----------------------------------------------------------------------------
    def _state_for(self, p, group):
        st = self.state[p]
        if not st:
            st["step"] = 0
            sd = torch.bfloat16 if p.dtype == torch.bfloat16 else torch.float32
            st["exp_avg"] = torch.zeros_like(p, dtype=sd, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=sd, memory_format=torch.preserve_format)
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            fused: dict[tuple, list] = {}
            for name, p in zip(group["param_names"], group["params"]):
                if p.grad is None:
                    continue
                st = self._state_for(p, group)
                st["step"] += 1
                step = st["step"]
                if p.dtype == torch.bfloat16:
                    fused.setdefault((step, p.device, p.grad.dtype), []).append((name, p, st))
                else:
                    self._fp32_step(p, st, lr, b1, b2, eps, wd, step)
            for (step, device, gdtype), items in fused.items():
                bc1 = 1.0 - b1**step
                bc2_sqrt = math.sqrt(1.0 - b2**step)
                step_size = lr / bc1
                wd_factor = 1.0 - lr * wd
                if device.type == "cuda":
                    self._cuda_step(gi, items, device, gdtype, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step)
                else:
                    skip = bool(self._skip.item()) if self._skip is not None else False
                    for name, p, st in items:
                        adamw_bf16_step_reference(
                            p, p.grad, st["exp_avg"], st["exp_avg_sq"], beta1=b1, beta2=b2, step_size=step_size,
                            bc2_sqrt=bc2_sqrt, eps=eps, wd_factor=wd_factor, key=self.key, step=step,
                            name_hash=param_name_hash(name),
                            grad_scale=None if self._grad_scale is None else self._grad_scale.cpu()[0], skip=skip,
                        )
        self._grad_scale = None
        return loss

    def _fp32_step(self, p, st, lr, b1, b2, eps, wd, step):
        g = p.grad.float()
        if self._grad_scale is not None:
            g = g * self._grad_scale.to(g.device)
        keep = None
        if self._skip is not None:
            keep = (self._skip.to(p.device) == 0).to(torch.float32)
        m, v = st["exp_avg"], st["exp_avg_sq"]
        m_new = m * b1 + g * (1 - b1)
        v_new = v * b2 + g * g * (1 - b2)
        denom = v_new.sqrt() / math.sqrt(1.0 - b2**step) + eps
        p_new = p.float() * (1.0 - lr * wd) - (lr / (1.0 - b1**step)) * m_new / denom
        if keep is not None:
            m_new = torch.lerp(m, m_new, keep)
            v_new = torch.lerp(v, v_new, keep)
            p_new = torch.lerp(p.float(), p_new, keep)
        m.copy_(m_new)
        v.copy_(v_new)
        p.copy_(p_new.to(p.dtype))

    def _cuda_step(self, gi, items, device, gdtype, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step):
        L = _lib.lib()
        params = [p for _, p, _ in items]
        grads = [p.grad.contiguous() for p in params]
        ms = [st["exp_avg"] for _, _, st in items]
        vs = [st["exp_avg_sq"] for _, _, st in items]
        hashes = [param_name_hash(n) for n, _, _ in items]
        table = self._tables.setdefault((gi, f"{device}:{gdtype}:{len(items)}"), _DeviceTable())
        tab, bstart, total_blocks = table.build(params, grads, ms, vs, hashes, device)
        base = tab.data_ptr()
        n = len(items)
        row = lambda i: ctypes.c_void_p(base + 8 * n * i)  # noqa: E731
        with torch.cuda.device(device):
            rc = L.halo_adamw_bf16_step(
                row(0), row(1), row(2), row(3), row(4), row(5), _lib.ptr(bstart), _lib.c_int(n),
                _lib.c_int(total_blocks), _lib.c_int(1 if gdtype == torch.float32 else 0),
                _lib.c_float(b1), _lib.c_float(b2), _lib.c_float(step_size), _lib.c_float(bc2_sqrt),
                _lib.c_float(eps), _lib.c_float(wd_factor), ctypes.c_ulonglong(self.key), ctypes.c_ulonglong(step),
                _lib.ptr(self._grad_scale), _lib.ptr(self._skip), _lib.stream_ptr(device),
            )
        _lib.check(rc, "halo_adamw_bf16_step")
        # the tables are device tensors: freeing them after the launch is stream-ordered and safe. Gradients
        # must NOT be kept alive here, or a whole extra set would survive zero_grad until the next step.


class GradNorm:
    """Global L2 norm of a set of gradients on the device, the clip coefficient and the non-finite
    flag derived from it - all without a host read."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.total_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.coef = torch.ones(1, dtype=torch.float32, device=self.device)
        self.skip = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.norm = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._table = _DeviceTable()
        self._partial = None

    def accumulate(self, grads: Iterable[torch.Tensor], first: bool = True) -> None:
        """``total_sq (+)= sum ||g||^2`` over ``grads`` (one dtype per call)."""
        grads = [g for g in grads if g is not None and g.numel() > 0]
        if self.device.type != "cuda":
            s = sum((g.float().pow(2).sum() for g in grads), torch.zeros((), dtype=torch.float32))
            self.total_sq[0] = s if first else self.total_sq[0] + s
            return
        if not grads:
            if first:
                self.total_sq.zero_()
            return
        by_dtype: dict[torch.dtype, list] = {}
        for g in grads:
            by_dtype.setdefault(g.dtype, []).append(g.contiguous())
        L = _lib.lib()
        for i, (dt, gs) in enumerate(by_dtype.items()):
            tab, bstart, total_blocks = _DeviceTable().build(gs, gs, gs, gs, [0] * len(gs), self.device)
            if self._partial is None or self._partial.numel() < total_blocks:
                self._partial = torch.empty(max(total_blocks, 1), dtype=torch.float32, device=self.device)
            n = len(gs)
            base = tab.data_ptr()
            rc = L.halo_sq_norm(
                ctypes.c_void_p(base + 8 * n * 1), ctypes.c_void_p(base + 8 * n * 4), _lib.ptr(bstart), _lib.c_int(n),
                _lib.c_int(total_blocks), _lib.c_int(1 if dt == torch.float32 else 0), _lib.ptr(self._partial),
                _lib.ptr(self.total_sq), _lib.c_int(0 if (first and i == 0) else 1), _lib.stream_ptr(self.device),
            )
            _lib.check(rc, "halo_sq_norm")

    def finish(self, max_norm: float) -> None:
        """coef = min(1, max_norm / (norm + 1e-6)); skip = norm is not finite."""
        if self.device.type != "cuda":
            norm = self.total_sq.sqrt()
            self.norm.copy_(norm)
            finite = torch.isfinite(norm)
            self.skip[0] = 0 if bool(finite) else 1
            c = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if (max_norm > 0 and bool(finite)) else torch.ones(1)
            self.coef.copy_(c)
            return
        rc = _lib.lib().halo_clip_coef(_lib.ptr(self.total_sq), _lib.c_float(max_norm), _lib.ptr(self.coef),
                                       _lib.ptr(self.skip), _lib.ptr(self.norm), _lib.stream_ptr(self.device))
        _lib.check(rc, "halo_clip_coef")
