"""Muon: momentum + Newton-Schulz orthogonalisation for 2-D hidden matrices, AdamW for everything
else (embeddings, head, norms, routers). Expert banks ``[E, out, in]`` are orthogonalised per
expert. bf16 weights are written back with the same keyed stochastic rounding as AdamWBF16, under
its own key so the two never share a noise stream (the role of halo/optimizers/muon.py)."""

from __future__ import annotations

import numpy as np
import torch

from .adamw_bf16 import param_name_hash, philox4x32_10, sr_key_pair

MUON_SR_KEY = 0x3A0B1D5
NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(g: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Approximate orthogonal factor of the last two dims (quintic iteration, fp32 or bf16 matmuls)."""
    a, b, c = NS_COEFFS
    x = g.to(torch.float32)
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.transpose(-1, -2)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        xxt = x @ x.transpose(-1, -2)
        x = a * x + (b * xxt + c * (xxt @ xxt)) @ x
    if transposed:
        x = x.transpose(-1, -2)
    return x


def _sr_to_bf16_(dst: torch.Tensor, value_fp32: torch.Tensor, key: int, step: int, name: str) -> None:
    n = value_fp32.numel()
    k0, k1 = sr_key_pair(key, step, param_name_hash(name))
    rnd = philox4x32_10(k0, k1, np.arange((n + 3) // 4, dtype=np.uint64)).reshape(-1)[:n]
    noise = torch.from_numpy((rnd & 0xFFFF).astype(np.int64)).to(value_fp32.device)
    bits = value_fp32.contiguous().view(torch.int32).reshape(-1) + noise.to(torch.int32)
    dst.reshape(-1).copy_((bits & -65536).view(torch.float32).to(torch.bfloat16))


class Muon(torch.optim.Optimizer):
    def __init__(self, params, lr=2e-2, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0,
                 adam_lr_ratio=0.015, adam_betas=(0.9, 0.95), adam_eps=1e-8):
        params = list(params)
        if params and isinstance(params[0], tuple):
            params = [{"params": [p for _, p in params], "param_names": [n for n, _ in params]}]
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      weight_decay=weight_decay, adam_lr_ratio=adam_lr_ratio,
                                      adam_betas=adam_betas, adam_eps=adam_eps))
        for g in self.param_groups:
            if "param_names" not in g:
                raise ValueError("Muon keys its stochastic rounding by parameter name: pass (name, param) pairs")

    @staticmethod
    def uses_muon(name: str, p: torch.Tensor) -> bool:
        return p.dim() >= 2 and not any(k in name for k in ("embed_tokens", "lm_head", "mlp.gate"))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            for name, p in zip(g["param_names"], g["params"]):
                if p.grad is None:
                    continue
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                grad = p.grad.float()
                if self.uses_muon(name, p):
                    buf = st.setdefault("momentum", torch.zeros_like(grad))
                    buf.mul_(g["momentum"]).add_(grad)
                    upd = grad.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                    o = newton_schulz(upd, g["ns_steps"])
                    scale = max(1.0, p.shape[-2] / p.shape[-1]) ** 0.5
                    new = p.float() * (1.0 - g["lr"] * g["weight_decay"]) - g["lr"] * scale * o
                else:
                    b1, b2 = g["adam_betas"]
                    m = st.setdefault("exp_avg", torch.zeros_like(grad))
                    v = st.setdefault("exp_avg_sq", torch.zeros_like(grad))
                    m.mul_(b1).add_(grad, alpha=1 - b1)
                    v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
                    t = st["step"]
                    denom = (v / (1 - b2**t)).sqrt_().add_(g["adam_eps"])
                    new = p.float() - g["lr"] * g["adam_lr_ratio"] * (m / (1 - b1**t)) / denom
                if p.dtype == torch.bfloat16:
                    _sr_to_bf16_(p.data, new, MUON_SR_KEY, st["step"], name)
                else:
                    p.copy_(new.to(p.dtype))
