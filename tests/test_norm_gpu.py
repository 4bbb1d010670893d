"""RMSNorm kernels (with and without the folded residual) against the PyTorch restatement."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("H", [256, 1024, 2048, 3072, 4096, 8192])
@pytest.mark.parametrize("rows", [1, 37, 1000])
def test_rms_norm_fwd_bwd(H, rows):
    from halo_b200.ops.norm import add_rms_norm, rms_norm, rms_norm_reference

    torch.manual_seed(0)
    x = torch.randn(rows, H, device="cuda").bfloat16()
    r = torch.randn(rows, H, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
    for use_res in (False, True):
        xa, ra, wa = x.clone().requires_grad_(), r.clone().requires_grad_(), w.clone().requires_grad_()
        xb, rb, wb = x.float().requires_grad_(), r.float().requires_grad_(), w.float().requires_grad_()
        if use_res:
            ya, ha = add_rms_norm(xa, ra, wa, 1e-6)
            yb, hb = rms_norm_reference(xb, wb, 1e-6, rb)
            g1, g2 = torch.randn_like(ya), torch.randn_like(ya)
            (ya.float() * g1.float()).sum().add((ha.float() * g2.float()).sum()).backward()
            (yb * g1.float()).sum().add((hb * g2.float()).sum()).backward()
        else:
            ya = rms_norm(xa, wa, 1e-6)
            yb = rms_norm_reference(xb, wb, 1e-6)
            g1 = torch.randn_like(ya)
            (ya.float() * g1.float()).sum().backward()
            (yb * g1.float()).sum().backward()
        assert (ya.float() - yb).abs().max().item() <= 3e-2 * yb.abs().max().item()
        assert (xa.grad.float() - xb.grad).abs().max().item() <= 3e-2 * xb.grad.abs().max().item() + 1e-3
        assert (wa.grad.float() - wb.grad).abs().max().item() <= 3e-2 * wb.grad.abs().max().item() + 1e-2
        if use_res:
            assert (ra.grad.float() - rb.grad).abs().max().item() <= 3e-2 * rb.grad.abs().max().item() + 1e-3
