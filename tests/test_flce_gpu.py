"""Fused linear + cross-entropy and the log-prob scorer against full-logits PyTorch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H,V,chunk", [(300, 256, 4096, 128), (1000, 512, 32000, 4096)])
def test_fused_linear_cross_entropy(T, H, V, chunk):
    from halo_b200.ops.cross_entropy import fused_linear_cross_entropy

    torch.manual_seed(0)
    h = torch.randn(T, H, device="cuda").bfloat16()
    w = (torch.randn(V, H, device="cuda") * 0.05).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    ha, wa = h.clone().requires_grad_(), w.clone().requires_grad_()
    loss = fused_linear_cross_entropy(ha, wa, labels, chunk_rows=chunk)
    loss.backward()
    hb, wb = h.float().requires_grad_(), w.float().requires_grad_()
    ref = torch.nn.functional.cross_entropy((hb @ wb.t()), labels, ignore_index=-100, reduction="sum") / (labels != -100).sum()
    ref.backward()
    assert abs(loss.item() - ref.item()) <= 2e-2 * abs(ref.item())
    assert (ha.grad.float() - hb.grad).abs().max().item() <= 5e-2 * hb.grad.abs().max().item() + 1e-6
    assert (wa.grad.float() - wb.grad).abs().max().item() <= 5e-2 * wb.grad.abs().max().item() + 1e-6


def test_linear_logprobs():
    from halo_b200.ops.cross_entropy import linear_logprobs

    torch.manual_seed(1)
    T, H, V = 500, 256, 8192
    h = torch.randn(T, H, device="cuda").bfloat16()
    w = (torch.randn(V, H, device="cuda") * 0.05).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    ha, wa = h.clone().requires_grad_(), w.clone().requires_grad_()
    logp, ent = linear_logprobs(ha, wa, labels, chunk_rows=200, want_entropy=True)
    g = torch.randn(T, device="cuda")
    (logp * g).sum().backward()
    hb, wb = h.float().requires_grad_(), w.float().requires_grad_()
    lp = torch.log_softmax(hb @ wb.t(), dim=-1)
    ref = lp.gather(-1, labels[:, None])[:, 0]
    (ref * g).sum().backward()
    ent_ref = -(lp.exp() * lp).sum(-1)
    assert (logp - ref).abs().max().item() <= 5e-2
    assert (ent - ent_ref).abs().max().item() <= 5e-2
    assert (ha.grad.float() - hb.grad).abs().max().item() <= 5e-2 * hb.grad.abs().max().item() + 1e-6
    assert (wa.grad.float() - wb.grad).abs().max().item() <= 5e-2 * wb.grad.abs().max().item() + 1e-6
