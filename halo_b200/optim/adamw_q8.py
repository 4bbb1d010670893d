"""AdamW with 8-bit moments and 24-bit weights: 5 bytes of state per parameter (bf16 parameter, 8-bit weight
correction, two 8-bit moment codes) instead of 6 with bf16 moments or 16 with fp32 master weights and moments.

* **Weights.** The model computes on the bf16 parameter ``p``; the optimizer's weight is
  ``w = p + c * ulp(p) / 256`` with a signed 8-bit ``c``: 16 significant bits, so updates far smaller than bf16's spacing
  accumulate instead of being rounded away (the reason the plain bf16 optimizer needs stochastic rounding of ``p``).
  ``p`` is always the nearest bf16 value of the updated weight; the correction is rounded stochastically, so even an update
  below 1/256 of the spacing moves the weight in expectation.
* **Moments.** Per group of 256 elements one fp32 scale and 8-bit codes on a square-root-spaced grid:
  ``m = sign(q) (|q| / 127)^2 m_scale`` and ``sqrt(v) = (q / 255)^2 v_scale``. Codes are rounded stochastically with
  Philox noise keyed by (optimizer key, step, parameter name) and the element offset, so a slowly decaying moment is
  unbiased rather than stuck on a grid point, runs are reproducible and resume exactly; a positive second moment never
  gets code 0.
* One launch steps every tensor of a parameter group; the clip coefficient and the skip flag are read on the device
  (same hand-off as :class:`halo_b200.optim.adamw_bf16.AdamWBF16`).

``adamw_q8_step_reference`` is the tensor-op statement of the kernel, bit for bit (the kernel file is compiled without
fused multiply-add contraction). Counterpart of the reference's FlashAdamW integration
(halo/optimizers/flash_adamw.py:1-97: 8-bit quantised moments plus compressed master weights, about 5 B/param).
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from halo_b200.ops import _lib

from .adamw_bf16 import SR_KEY, param_name_hash, philox4x32_10, sr_key_pair

GROUP = 256


def n_groups(numel: int) -> int:
    return (numel + GROUP - 1) // GROUP


def spacing_256th(p_f32: torch.Tensor) -> torch.Tensor:
    """``ulp_bf16(p) / 256`` as fp32: a power of two read off the exponent field (0 for values below 2^-111)."""
    e = (p_f32.contiguous().view(torch.int32) >> 23) & 0xFF
    bits = torch.where(e > 15, (e - 15) << 23, torch.zeros_like(e))
    return bits.view(torch.float32)


def master_weight(p: torch.Tensor, corr: torch.Tensor) -> torch.Tensor:
    """The optimizer's fp32 weight of a bf16 parameter and its correction."""
    pf = p.detach().float()
    return pf + corr.float() * spacing_256th(pf)


def dequantize_moments(mq, vq, m_scale, v_scale):
    """fp32 ``(m, v)`` of flat code tensors."""
    n = mq.numel()
    ms = m_scale.repeat_interleave(GROUP)[:n]
    vs = v_scale.repeat_interleave(GROUP)[:n]
    rm = mq.reshape(-1).to(torch.int32).abs().float() / 127.0
    m = (rm * rm) * ms
    m = torch.where(mq.reshape(-1) < 0, -m, m)
    rv = vq.reshape(-1).float() / 255.0
    s = (rv * rv) * vs
    return m, s * s


MIN_SCALE = 1e-30     # kQ8MinScale of the kernel


def _sqrt32(x: torch.Tensor) -> torch.Tensor:
    """Correctly rounded fp32 square root (what ``sqrtf`` gives on the device): the CPU's vectorised fp32 ``sqrt`` is off
    by an ulp on a fraction of a percent of inputs; rounding the fp64 root to fp32 is exact."""
    return x.double().sqrt().float()


def adamw_q8_step_reference(p, g, corr, mq, vq, m_scale, v_scale, *, beta1, beta2, step_size, bc2_sqrt, eps, wd_factor, key, step,
                            name_hash, grad_scale=None, skip=False):
    """Bit-exact CPU twin of ``adamw_q8_kernel`` for one tensor (updates every state tensor in place)."""
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
    pf = p.detach().reshape(-1).float()
    w = pf + corr.reshape(-1).float() * spacing_256th(pf)
    m, v_from_codes = dequantize_moments(mq, vq, m_scale, v_scale)
    omb1 = f32(1.0 - float(np.float32(beta1)))
    omb2 = f32(1.0 - float(np.float32(beta2)))
    mn = m * f32(beta1) + gf * omb1
    vn = v_from_codes * f32(beta2) + (gf * gf) * omb2
    sn = _sqrt32(vn)
    denom = sn * (f32(1.0) / f32(bc2_sqrt)) + f32(eps)
    wn = w * f32(wd_factor) - (f32(step_size) * mn) / denom
    # group maxima
    G = n_groups(n)
    pad = G * GROUP - n
    m_max = torch.nn.functional.pad(mn.abs(), (0, pad)).view(G, GROUP).max(dim=1).values
    s_max = torch.nn.functional.pad(sn, (0, pad)).view(G, GROUP).max(dim=1).values
    mm = m_max.repeat_interleave(GROUP)[:n]
    sm = s_max.repeat_interleave(GROUP)[:n]
    k0, k1 = sr_key_pair(key, step, name_hash)
    quads = (n + 3) // 4
    rnd = philox4x32_10(k0, k1, np.arange(quads, dtype=np.uint64)).reshape(-1)[:n]
    rnd_t = torch.from_numpy(rnd.astype(np.int64))
    um = (rnd_t & 0x7FF).float() / 2048.0
    uv = ((rnd_t >> 11) & 0x7FF).float() / 2048.0
    uc = (rnd_t >> 22).float() / 1024.0
    # one reciprocal per group; groups whose largest moment is below MIN_SCALE keep their scale and store zero codes
    inv_mm = torch.where(mm > f32(MIN_SCALE), f32(1.0) / torch.where(mm > 0, mm, torch.ones_like(mm)), torch.zeros_like(mm))
    qm = torch.floor(_sqrt32(mn.abs() * inv_mm) * 127.0 + um).clamp(max=127.0)
    qm = torch.where(inv_mm > 0, qm, torch.zeros_like(qm))
    qm = torch.where(mn < 0, -qm, qm)
    inv_sm = torch.where(sm > f32(MIN_SCALE), f32(1.0) / torch.where(sm > 0, sm, torch.ones_like(sm)), torch.zeros_like(sm))
    qv = torch.floor(_sqrt32(sn * inv_sm) * 255.0 + uv).clamp(min=1.0, max=255.0)
    qv = torch.where((inv_sm > 0) & (sn > 0), qv, torch.zeros_like(qv))
    pn = wn.bfloat16()
    pnf = pn.float()
    st = spacing_256th(pnf)
    safe_st = torch.where(st > 0, st, torch.ones_like(st))
    c = torch.floor((wn - pnf) / safe_st + uc).clamp(min=-128.0, max=127.0)
    c = torch.where(st > 0, c, torch.zeros_like(c))
    p.detach().reshape(-1).copy_(pn)
    corr.reshape(-1).copy_(c.to(torch.int8))
    mq.reshape(-1).copy_(qm.to(torch.int8))
    vq.reshape(-1).copy_(qv.to(torch.uint8))
    m_scale.copy_(m_max)
    v_scale.copy_(s_max)


class _Q8Table:
    def __init__(self):
        self.sig = None
        self.tensors = None

    def build(self, items, grads, hashes, device):
        L = _lib.lib()
        epb = int(L.halo_adam_q8_elems_per_block())
        sig = tuple((p.data_ptr(), g.data_ptr(), st["corr"].data_ptr(), p.numel()) for (_, p, st), g in zip(items, grads))
        if sig == self.sig:
            return self.tensors
        n = len(items)
        arr = np.zeros((9, n), dtype=np.uint64)
        blocks = [0]
        for i, ((_, p, st), g, h) in enumerate(zip(items, grads, hashes)):
            arr[:, i] = (p.data_ptr(), g.data_ptr(), st["corr"].data_ptr(), st["exp_avg_q"].data_ptr(), st["exp_avg_sq_q"].data_ptr(),
                         st["exp_avg_scale"].data_ptr(), st["exp_avg_sq_scale"].data_ptr(), p.numel(), h)
            blocks.append(blocks[-1] + (p.numel() + epb - 1) // epb)
        tab = torch.from_numpy(arr.view(np.int64)).to(device)
        bstart = torch.tensor(blocks, dtype=torch.int32).to(device)
        self.sig, self.tensors = sig, (tab, bstart, blocks[-1])
        return self.tensors


class AdamWQ8(torch.optim.Optimizer):
    """``params``: ``(name, parameter)`` pairs or param-group dicts with ``params`` and ``param_names``. bf16 parameters
    take the 5-byte state; parameters of another dtype (fp32 norms in a mixed model) take plain fp32 AdamW."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01, key: int = SR_KEY):
        if lr < 0.0 or eps < 0.0 or not 0.0 <= betas[0] < 1.0 or not 0.0 <= betas[1] < 1.0:
            raise ValueError("invalid AdamWQ8 hyper-parameters")
        params = list(params)
        if params and isinstance(params[0], tuple):
            params = [{"params": [p for _, p in params], "param_names": [n for n, _ in params]}]
        super().__init__(params, {"lr": lr, "betas": betas, "eps": eps, "weight_decay": weight_decay})
        for group in self.param_groups:
            if "param_names" not in group or len(group["param_names"]) != len(group["params"]):
                raise ValueError("AdamWQ8 keys its rounding noise by parameter name: build it from (name, param) pairs or "
                                 "groups carrying 'param_names'")
        self.key = key
        self._grad_scale: torch.Tensor | None = None
        self._skip: torch.Tensor | None = None
        self._tables: dict = {}

    def defer_grad_scale(self, scale: torch.Tensor | None) -> None:
        self._grad_scale = None if scale is None else scale.detach().to(torch.float32).reshape(1)

    def arm_skip(self, flag: torch.Tensor | None) -> None:
        self._skip = None if flag is None else flag.reshape(1)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._grad_scale = None
        super().zero_grad(set_to_none=set_to_none)

    def _state_for(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            if p.dtype == torch.bfloat16:
                G = n_groups(p.numel())
                st["corr"] = torch.zeros(p.numel(), dtype=torch.int8, device=p.device)
                st["exp_avg_q"] = torch.zeros(p.numel(), dtype=torch.int8, device=p.device)
                st["exp_avg_sq_q"] = torch.zeros(p.numel(), dtype=torch.uint8, device=p.device)
                st["exp_avg_scale"] = torch.zeros(G, dtype=torch.float32, device=p.device)
                st["exp_avg_sq_scale"] = torch.zeros(G, dtype=torch.float32, device=p.device)
            else:
                st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
        return st

    def load_state_dict(self, state_dict) -> None:
        """The base class casts floating-point state to the parameter's dtype, which would round the fp32 group scales
        (and the fp32 moments of non-bf16 parameters) to bf16: they are restored from ``state_dict`` at full precision."""
        super().load_state_dict(state_dict)
        ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        params = [p for g in self.param_groups for p in g["params"]]
        for pid, p in zip(ids, params):
            saved = state_dict["state"].get(pid)
            if saved is None:
                continue
            for key, value in saved.items():
                if torch.is_tensor(value) and value.is_floating_point():
                    self.state[p][key] = value.detach().clone().to(p.device)

    def state_bytes_per_param(self) -> float:
        total = numel = 0
        for st_p, st in self.state.items():
            numel += st_p.numel()
            total += st_p.numel() * st_p.element_size() + sum(t.numel() * t.element_size() for t in st.values() if torch.is_tensor(t))
        return total / max(numel, 1)

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
                st = self._state_for(p)
                st["step"] += 1
                step = st["step"]
                if p.dtype == torch.bfloat16:
                    if not p.is_contiguous():
                        raise ValueError(f"{name}: the 8-bit-state optimizer needs contiguous parameters")
                    fused.setdefault((step, p.device, p.grad.dtype), []).append((name, p, st))
                else:
                    self._fp32_step(p, st, lr, b1, b2, eps, wd, step)
            for (step, device, gdtype), items in fused.items():
                bc1 = 1.0 - b1**step
                bc2_sqrt = math.sqrt(1.0 - b2**step)
                step_size, wd_factor = lr / bc1, 1.0 - lr * wd
                if device.type == "cuda":
                    self._cuda_step(gi, items, device, gdtype, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step)
                else:
                    skip = bool(self._skip.item()) if self._skip is not None else False
                    for name, p, st in items:
                        adamw_q8_step_reference(
                            p, p.grad, st["corr"], st["exp_avg_q"], st["exp_avg_sq_q"], st["exp_avg_scale"], st["exp_avg_sq_scale"],
                            beta1=b1, beta2=b2, step_size=step_size, bc2_sqrt=bc2_sqrt, eps=eps, wd_factor=wd_factor, key=self.key,
                            step=step, name_hash=param_name_hash(name),
                            grad_scale=None if self._grad_scale is None else self._grad_scale.cpu()[0], skip=skip)
        self._grad_scale = None
        return loss

    def _fp32_step(self, p, st, lr, b1, b2, eps, wd, step):
        g = p.grad.float()
        if self._grad_scale is not None:
            g = g * self._grad_scale.to(g.device)
        keep = (self._skip.to(p.device) == 0).to(torch.float32) if self._skip is not None else None
        m, v = st["exp_avg"], st["exp_avg_sq"]
        m_new = m * b1 + g * (1 - b1)
        v_new = v * b2 + g * g * (1 - b2)
        denom = v_new.sqrt() / math.sqrt(1.0 - b2**step) + eps
        p_new = p.float() * (1.0 - lr * wd) - (lr / (1.0 - b1**step)) * m_new / denom
        if keep is not None:
            m_new, v_new, p_new = torch.lerp(m, m_new, keep), torch.lerp(v, v_new, keep), torch.lerp(p.float(), p_new, keep)
        m.copy_(m_new)
        v.copy_(v_new)
        p.copy_(p_new.to(p.dtype))

    def _cuda_step(self, gi, items, device, gdtype, b1, b2, step_size, bc2_sqrt, eps, wd_factor, step):
        L = _lib.lib()
        grads = [p.grad.contiguous() for _, p, _ in items]
        hashes = [param_name_hash(n) for n, _, _ in items]
        table = self._tables.setdefault((gi, f"{device}:{gdtype}:{len(items)}"), _Q8Table())
        tab, bstart, total_blocks = table.build(items, grads, hashes, device)
        with torch.cuda.device(device):
            rc = L.halo_adamw_q8_step(
                _lib.ptr(tab), _lib.ptr(bstart), _lib.c_int(len(items)), _lib.c_int(total_blocks),
                _lib.c_int(1 if gdtype == torch.float32 else 0), _lib.c_float(b1), _lib.c_float(b2), _lib.c_float(step_size),
                _lib.c_float(bc2_sqrt), _lib.c_float(eps), _lib.c_float(wd_factor), ctypes.c_ulonglong(self.key),
                ctypes.c_ulonglong(step), _lib.ptr(self._grad_scale), _lib.ptr(self._skip), _lib.stream_ptr(device))
        _lib.check(rc, "halo_adamw_q8_step")
