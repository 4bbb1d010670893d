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


def _row_rel_err(a, b):
    """Largest per-row relative error: ||a_row - b_row|| / (||b_row|| + 2 % of the mean row norm). A row is judged
    against its own size, so a small row cannot hide behind the tensor's largest value; the floor keeps rows that are
    exactly zero in the reference (a document's first query has no gradient) from dividing by nothing."""
    a, b = a.float(), b.float()
    norms = b.norm(dim=-1)
    return ((a - b).norm(dim=-1) / (norms + 0.02 * norms.mean())).max().item()


@pytest.mark.parametrize("lens,scale_logits,bwd_variant", [
    ([16384, 500], 1.0, 2),            # a 16k-token document: 256 key tiles per query tile, every pipeline slot reused many times
    ([4096, 3000, 1096], 8.0, 2),      # logits x8: row maxima jump by far more than 2^8 between tiles (the lazy rescale fires)
    ([2500, 1300], 1.0, 1),            # the first backward form stays correct beside the double-buffered one
])
def test_flash_attention_long_documents_and_large_logits(lens, scale_logits, bwd_variant, monkeypatch):
    import subprocess
    import sys

    if bwd_variant != 2:
        # the variant is read once per process: check the other one in a child
        code = ("import os, sys; os.environ['HALO_ATTN_BWD_VARIANT']='1'; sys.path.insert(0, '.');"
                "import tests.test_attention_gpu as t; t._long_case(%r, %r)" % (lens, scale_logits))
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        return
    _long_case(lens, scale_logits)


def _long_case(lens, scale_logits):
    from halo_b200.ops import _lib
    from halo_b200.ops.attention import attention_reference, build_plan, flash_attention

    Hq, Hkv = 4, 2
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    q, k, v = _mk(cu[-1], Hq, Hkv, seed=3)
    q = (q.float() * scale_logits ** 0.5).bfloat16()
    k = (k.float() * scale_logits ** 0.5).bfloat16()
    plan = build_plan(cu, device="cuda")
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    o = flash_attention(qg, kg, vg, plan, Hq, Hkv)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    # the fp32 oracle, one document at a time (a 16k x 16k score matrix per head fits; all heads at once would not)
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    o_ref = attention_reference(qr, kr, vr, cu, Hq, Hkv)
    o_ref.backward(do.float())
    assert _row_rel_err(o, o_ref) < 2e-2
    assert _row_rel_err(vg.grad, vr.grad) < 3e-2
    if scale_logits == 1.0:
        assert _row_rel_err(qg.grad, qr.grad) < 4e-2
        assert _row_rel_err(kg.grad, kr.grad) < 4e-2
    else:
        # nearly one-hot rows: dS = P (dP - delta) cancels almost completely for the winning key, and delta is formed from
        # the bf16 output, so single rows of dQ / dK carry the rounding of O at full size (any bf16 flash backward does);
        # the gradients as a whole must still agree
        for got, want, name in ((qg.grad, qr.grad, "dq"), (kg.grad, kr.grad, "dk")):
            rel = ((got.float() - want).norm() / want.norm()).item()
            assert rel < 5e-2, (name, rel)


@pytest.mark.parametrize("lens,window", [
    ([700, 300, 1048], 256),      # several documents, windows shorter than most of them
    ([2048], 128),                # every key tile is cut by the diagonal or by a window edge
    ([5000, 120], 1024),
    ([333], 4096),                # a window longer than the document: plain causal attention
    ([1500, 777], 100),           # a window that is no multiple of the tile sizes
])
def test_flash_attention_sliding_window(lens, window):
    from halo_b200.ops import _lib
    from halo_b200.ops.attention import attention_reference, build_plan, flash_attention

    Hq, Hkv = 4, 2
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    q, k, v = _mk(cu[-1], Hq, Hkv, seed=7)
    plan = build_plan(cu, device="cuda", window=window)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    o = flash_attention(qg, kg, vg, plan, Hq, Hkv)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    o_ref = attention_reference(qr, kr, vr, cu, Hq, Hkv, window=window)
    o_ref.backward(do.float())
    assert _row_rel_err(o, o_ref) < 2e-2
    assert _row_rel_err(vg.grad, vr.grad) < 3e-2
    assert _row_rel_err(qg.grad, qr.grad) < 4e-2
    assert _row_rel_err(kg.grad, kr.grad) < 4e-2
    # the window changes the result (unless it covers the whole document)
    if window < max(lens):
        full = flash_attention(q, k, v, build_plan(cu, device="cuda"), Hq, Hkv)
        assert (full.float() - o.float()).abs().max().item() > 1e-2


@pytest.mark.parametrize("lens,window", [([700, 300, 1048], 0), ([1500, 777], 200), ([130], 0)])
def test_flash_attention_sinks(lens, window):
    """One logit per head in every row's softmax: output, dq / dk / dv and the gradient of the logits themselves."""
    from halo_b200.ops import _lib
    from halo_b200.ops.attention import attention_reference, build_plan, flash_attention

    Hq, Hkv = 4, 2
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    q, k, v = _mk(cu[-1], Hq, Hkv, seed=11)
    # logits that matter: scores of unit-variance inputs at scale 128^-0.5 have a standard deviation near 1
    sinks = torch.tensor([2.0, -1.0, 0.5, 4.0], device="cuda")
    plan = build_plan(cu, device="cuda", window=window)
    qg, kg, vg, sg = (t.clone().requires_grad_() for t in (q, k, v, sinks))
    o = flash_attention(qg, kg, vg, plan, Hq, Hkv, sinks=sg)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    qr, kr, vr, sr = (t.float().requires_grad_() for t in (q, k, v, sinks))
    o_ref = attention_reference(qr, kr, vr, cu, Hq, Hkv, window=window, sinks=sr)
    o_ref.backward(do.float())
    assert _row_rel_err(o, o_ref) < 2e-2
    assert _row_rel_err(vg.grad, vr.grad) < 3e-2
    assert _row_rel_err(qg.grad, qr.grad) < 4e-2
    assert _row_rel_err(kg.grad, kr.grad) < 4e-2
    assert ((sg.grad - sr.grad).abs() / (sr.grad.abs() + 0.02 * sr.grad.abs().mean())).max().item() < 3e-2
    # the sinks take mass: the output differs from the sink-free one
    plain = flash_attention(q, k, v, plan, Hq, Hkv)
    assert (plain.float() - o.float()).abs().max().item() > 1e-2


def test_flash_attention_heads_of_64_run_zero_padded():
    from halo_b200.ops import _lib
    from halo_b200.ops.attention import attention_reference, build_plan, flash_attention

    Hq, Hkv, D = 8, 2, 64
    cu = [0, 400, 1000, 1111]
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(cu[-1], Hq * D, device="cuda", generator=g).bfloat16()
    k = torch.randn(cu[-1], Hkv * D, device="cuda", generator=g).bfloat16()
    v = torch.randn(cu[-1], Hkv * D, device="cuda", generator=g).bfloat16()
    sinks = torch.linspace(-1, 3, Hq, device="cuda")
    plan = build_plan(cu, device="cuda", window=128)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    o = flash_attention(qg, kg, vg, plan, Hq, Hkv, sinks=sinks)
    assert o.shape == (cu[-1], Hq * D)
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    o_ref = attention_reference(qr, kr, vr, cu, Hq, Hkv, window=128, sinks=sinks)
    o_ref.backward(do.float())
    assert _row_rel_err(o, o_ref) < 2e-2
    assert _row_rel_err(vg.grad, vr.grad) < 3e-2
    assert _row_rel_err(qg.grad, qr.grad) < 4e-2
    assert _row_rel_err(kg.grad, kr.grad) < 4e-2


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
