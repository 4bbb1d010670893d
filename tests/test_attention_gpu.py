"""tcgen05 flash attention (packed, causal, GQA) against an fp32 PyTorch attention, fwd and bwd."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(T, Hq, Hkv, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn(T, Hq * 128, device="cuda", generator=g)).bfloat16()
    k = (torch.randn(T, Hkv * 128, device="cuda", generator=g)).bfloat16()
    v = (torch.randn(T, Hkv * 128, device="cuda", generator=g)).bfloat16()
    return q, k, v


def _close(a, b, tol, name):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * ref + 1e-3, f"{name}: max err {err} vs ref max {ref}"


@pytest.mark.parametrize("lens,Hq,Hkv", [
    ([128], 1, 1),
    ([256], 2, 1),
    ([100], 2, 2),
    ([300, 77, 515], 4, 2),
    ([1024, 33, 1, 640], 8, 2),
])
def test_flash_attention_fwd_bwd(lens, Hq, Hkv):
    from halo_b200.ops import _lib
    from halo_b200.ops.attention import attention_reference, build_plan, flash_attention

    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    q, k, v = _mk(T, Hq, Hkv)
    plan = build_plan(cu, device="cuda")
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    o = flash_attention(qg, kg, vg, plan, Hq, Hkv)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    o_ref = attention_reference(qr, kr, vr, cu, Hq, Hkv)
    _close(o, o_ref, 2e-2, "out")
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    o_ref.backward(do.float())
    _close(qg.grad, qr.grad, 3e-2, "dq")
    _close(kg.grad, kr.grad, 3e-2, "dk")
    _close(vg.grad, vr.grad, 3e-2, "dv")


def test_rope_attention_fused_matches_reference():
    from halo_b200.ops.attention import build_plan, rope_attention
    from halo_b200.ops.rope import rope_table

    Hq, Hkv, lens = 4, 2, [200, 312]
    cu = [0, 200, 512]
    T = 512
    torch.manual_seed(0)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device="cuda").bfloat16()
    wq = (1 + 0.1 * torch.randn(128, device="cuda")).bfloat16()
    wk = (1 + 0.1 * torch.randn(128, device="cuda")).bfloat16()
    pos = torch.cat([torch.arange(n, device="cuda") for n in lens])
    table = rope_table(pos, 128, 1e6)
    table_cpu = rope_table(pos.cpu(), 128, 1e6)
    assert (table.cpu() - table_cpu).abs().max().item() < 1e-2
    plan = build_plan(cu, device="cuda")
    a = qkv.clone().requires_grad_()
    wqa, wka = wq.clone().requires_grad_(), wk.clone().requires_grad_()
    o = rope_attention(a, wqa, wka, table, plan, Hq, Hkv)
    do = torch.randn_like(o)
    o.backward(do)
    # oracle: same math on CPU in fp32 (weights/inputs as fp32 leaves)
    b = qkv.cpu().float().requires_grad_()
    wqb, wkb = wq.cpu().float().requires_grad_(), wk.cpu().float().requires_grad_()
    cplan = build_plan(cu)
    o_ref = rope_attention(b, wqb, wkb, table_cpu, cplan, Hq, Hkv)
    o_ref.backward(do.cpu().float())
    _close(o.cpu(), o_ref, 3e-2, "out")
    _close(a.grad.cpu(), b.grad, 4e-2, "dqkv")
    _close(wqa.grad.cpu(), wqb.grad, 5e-2, "dwq")
    _close(wka.grad.cpu(), wkb.grad, 5e-2, "dwk")
