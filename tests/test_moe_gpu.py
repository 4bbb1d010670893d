"""Router top-k, routing sort, dispatch / grouped FFN / combine against the per-expert PyTorch loop."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol, name):
    err = (a.float() - b.float()).abs().max().item()
    ref = b.float().abs().max().item()
    assert err <= tol * ref + 1e-3, f"{name}: max err {err} vs ref max {ref}"


@pytest.mark.parametrize("T,E,k", [(5, 32, 2), (1000, 128, 8), (333, 64, 4)])
def test_router_topk(T, E, k):
    from halo_b200.ops.moe import router_topk, router_topk_reference

    torch.manual_seed(0)
    logits = torch.randn(T, E, device="cuda")
    a = logits.clone().requires_grad_()
    idx, w = router_topk(a, k, True)
    b = logits.clone().requires_grad_()
    idx_r, w_r = router_topk_reference(b, k, True)
    assert torch.equal(idx.long().sort(-1).values, idx_r.long().sort(-1).values)
    _close(w.sort(-1).values, w_r.sort(-1).values, 1e-4, "weights")
    g = torch.randn_like(w)
    # align slot order before comparing gradients
    order = idx.long().argsort(-1)
    order_r = idx_r.long().argsort(-1)
    (w.gather(-1, order) * g).sum().backward()
    (w_r.gather(-1, order_r) * g).sum().backward()
    _close(a.grad, b.grad, 1e-3, "dlogits")


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("T,H,F,E,k", [(64, 256, 128, 8, 2), (777, 512, 256, 16, 4), (4096, 2048, 768, 32, 8)])
def test_moe_experts_fwd_bwd(T, H, F, E, k, fused):
    """``fused``: token movement inside the GEMM kernels (push warps + arrival-gated tiles, scatter epilogue) against
    the separate push / pull kernels; both against the per-expert fp32 loop."""
    from halo_b200.ops import _lib
    from halo_b200.ops.moe import LocalTransport, moe_experts, moe_ffn_reference

    transport = LocalTransport()
    transport.fused = fused

    torch.manual_seed(1)
    x = torch.randn(T, H, device="cuda").bfloat16()
    wgu = (torch.randn(E, 2 * F, H, device="cuda") * 0.05).bfloat16()
    wd = (torch.randn(E, H, F, device="cuda") * 0.05).bfloat16()
    scores = torch.rand(T, E, device="cuda")
    w, idx = torch.topk(scores, k, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).float()
    idx = idx.to(torch.int32)

    xa, wa, wgua, wda = (t.clone().requires_grad_() for t in (x, w, wgu, wd))
    out = moe_experts(xa, idx, wa, wgua, wda, transport)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    xb, wb, wgub, wdb = (t.float().requires_grad_() for t in (x, w, wgu, wd))
    ref = moe_ffn_reference(xb, idx, wb, wgub, wdb)
    _close(out, ref, 3e-2, "out")
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    _close(xa.grad, xb.grad, 4e-2, "dx")
    _close(wa.grad, wb.grad, 4e-2, "dw_route")
    _close(wgua.grad, wgub.grad, 4e-2, "dw_gate_up")
    _close(wda.grad, wdb.grad, 4e-2, "dw_down")


@pytest.mark.parametrize("T,H,F,E,k", [(64, 256, 128, 8, 2), (777, 512, 256, 16, 4), (3000, 1024, 512, 32, 4)])
def test_biased_clamped_glu_experts_fwd_bwd(T, H, F, E, k):
    """Experts with bias vectors around a clamped GLU on the grouped kernels (bias / activation row kernels between the
    products) against the dense fp32 form: output and every gradient, the two bias banks' included."""
    from halo_b200.ops import _lib
    from halo_b200.ops.biased_glu_experts import GLU_ALPHA, biased_glu_experts_reference
    from halo_b200.ops.moe import LocalTransport, moe_experts

    torch.manual_seed(2)
    x = torch.randn(T, H, device="cuda").bfloat16()
    wgu = (torch.randn(E, 2 * F, H, device="cuda") * 0.08).bfloat16()      # pre-activations of a few units: both clamps bite
    wd = (torch.randn(E, H, F, device="cuda") * 0.05).bfloat16()
    bgu = (torch.randn(E, 2 * F, device="cuda") * 0.5).bfloat16()
    bd = (torch.randn(E, H, device="cuda") * 0.5).bfloat16()
    limit = 2.0
    scores = torch.rand(T, E, device="cuda")
    w, idx = torch.topk(scores, k, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).float()
    idx = idx.to(torch.int32)

    leaves = [t.clone().requires_grad_() for t in (x, w, wgu, wd, bgu, bd)]
    xa, wa, wgua, wda, bgua, bda = leaves
    out = moe_experts(xa, idx, wa, wgua, wda, LocalTransport(), glu=(bgua, bda, limit, GLU_ALPHA))
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    refs = [t.float().requires_grad_() for t in (x, w, wgu, wd, bgu, bd)]
    xb, wb, wgub, wdb, bgub, bdb = refs
    # the oracle rounds the pre-activations where the kernels store them, so both clamp the same elements
    ref = biased_glu_experts_reference(xb, idx, wb, wgub, bgub, wdb, bdb, limit, stored_dtype=torch.bfloat16)
    _close(out, ref, 3e-2, "out")
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    # the clamps make the function discontinuous in its gradient: where a pre-activation lands within one bf16 step of
    # the limit, two correct summation orders can clamp differently, and ONE such element changes a whole row of a
    # gradient by a visible amount. Among millions of elements a handful do, so gradients are compared by their norm
    # (every systematic error shows there) and the largest single deviation only has to stay below a quarter of the
    # largest entry
    names = ("dx", "dw_route", "dw_gate_up", "dw_down", "db_gate_up", "db_down")
    for got, want, name in zip(leaves, refs, names):
        assert got.grad is not None, name
        diff = (got.grad.float() - want.grad.float())
        assert diff.norm().item() <= 2e-2 * want.grad.float().norm().item() + 1e-6, (name, diff.norm().item(), want.grad.norm().item())
        assert diff.abs().max().item() <= 0.25 * want.grad.abs().max().item() + 1e-3, name
    # a recomputation that skips its output still gives the same gradients
    again = [t.detach().clone().requires_grad_() for t in (x, w, wgu, wd, bgu, bd)]      # w became a leaf of the oracle's graph above
    out2 = moe_experts(again[0], idx, again[1], again[2], again[3], LocalTransport(), skip_output=True,
                       glu=(again[4], again[5], limit, GLU_ALPHA))
    out2.backward(g)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    for a, b2, name in zip(again, leaves, names):
        assert a.grad is not None, f"{name}: no gradient from the output-skipping form"
        assert torch.equal(a.grad, b2.grad), (name, (a.grad.float() - b2.grad.float()).abs().max().item())


def test_fused_moe_calls_in_a_row_share_one_control_block():
    """Several layers' worth of calls through one transport (forward, a recomputation that skips its output, backward):
    the control block's call numbers, buffer parities and arrival counters must carry over from call to call."""
    from halo_b200.ops import _lib
    from halo_b200.ops.moe import LocalTransport, moe_experts, moe_ffn_reference

    torch.manual_seed(5)
    T, H, F, E, k = 1500, 512, 256, 32, 4
    transport = LocalTransport()
    transport.fused = True
    wgu = (torch.randn(E, 2 * F, H, device="cuda") * 0.05).bfloat16()
    wd = (torch.randn(E, H, F, device="cuda") * 0.05).bfloat16()
    for step in range(5):
        x = torch.randn(T - 100 * step, H, device="cuda").bfloat16()
        w, idx = torch.topk(torch.rand(x.shape[0], E, device="cuda"), k, dim=-1)
        w = (w / w.sum(-1, keepdim=True)).float()
        idx = idx.to(torch.int32)
        with torch.no_grad():
            first = moe_experts(x, idx, w, wgu, wd, transport)
        xa, wgua = x.clone().requires_grad_(), wgu.clone().requires_grad_()
        out = moe_experts(xa, idx, w, wgua, wd, transport, skip_output=step % 2 == 1)
        g = torch.randn_like(first)
        out.backward(g)
        torch.cuda.synchronize()
        assert _lib.read_status() == 0
        xb, wgub = x.float().requires_grad_(), wgu.float().requires_grad_()
        ref = moe_ffn_reference(xb, idx, w, wgub, wd.float())
        ref.backward(g.float())
        _close(first, ref, 3e-2, f"out, call {step}")
        _close(xa.grad, xb.grad, 4e-2, f"dx, call {step}")
        _close(wgua.grad, wgub.grad, 4e-2, f"dw_gate_up, call {step}")
    assert transport.seq == 15


def test_moe_empty_experts():
    """Experts that receive no token get a zero weight gradient and do not disturb the others."""
    from halo_b200.ops.moe import moe_experts, moe_ffn_reference

    torch.manual_seed(2)
    T, H, F, E, k = 200, 256, 128, 16, 2
    x = torch.randn(T, H, device="cuda").bfloat16()
    wgu = (torch.randn(E, 2 * F, H, device="cuda") * 0.05).bfloat16().requires_grad_()
    wd = (torch.randn(E, H, F, device="cuda") * 0.05).bfloat16().requires_grad_()
    idx = torch.randint(0, 4, (T, k), device="cuda", dtype=torch.int32)  # experts 4..15 stay empty
    idx[:, 1] = (idx[:, 0] + 1) % 4
    w = torch.full((T, k), 0.5, device="cuda")
    out = moe_experts(x, idx, w, wgu, wd)
    ref = moe_ffn_reference(x.float(), idx, w, wgu.float(), wd.float())
    _close(out, ref, 3e-2, "out")
    out.float().sum().backward()
    assert torch.all(wgu.grad[4:] == 0) and torch.all(wd.grad[4:] == 0)
    assert torch.isfinite(wgu.grad).all() and torch.isfinite(wd.grad).all()


@pytest.mark.gpu
def test_router_topk_selection_bias_matches_reference():
    torch.manual_seed(3)
    logits = torch.randn(1000, 128, device="cuda")
    bias = torch.randn(128, device="cuda") * 0.05
    from halo_b200.ops.moe import router_topk, router_topk_reference

    idx, w = router_topk(logits, 8, True, bias)
    ridx, rw = router_topk_reference(logits, 8, True, bias)
    assert torch.equal(idx.sort(-1).values, ridx.sort(-1).values)
    assert torch.allclose(w.sum(-1), torch.ones_like(w.sum(-1)), atol=1e-5)
    assert torch.allclose(w.sort(-1).values, rw.sort(-1).values, atol=1e-5)
