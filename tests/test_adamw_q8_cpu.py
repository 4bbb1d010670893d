"""The 8-bit-state AdamW (5 bytes per parameter): its tensor-op statement against fp32 AdamW on long runs, the 24-bit
weight representation, the moment codes, reproducibility and resume."""

import math

import pytest
import torch


def test_weight_correction_represents_sixteen_significant_bits():
    from halo_b200.optim.adamw_q8 import master_weight, spacing_256th

    p = torch.tensor([1.0, 1.5, -0.37, 3e-3, 1e4, 0.0], dtype=torch.bfloat16)
    st = spacing_256th(p.float())
    # bf16 spacing at 1.0 is 2^-7: a 256th of it is 2^-15
    assert st[0].item() == 2.0**-15 and st[5].item() == 0.0
    corr = torch.tensor([100, -128, 127, 5, -1, 9], dtype=torch.int8)
    w = master_weight(p, corr)
    assert w[0].item() == 1.0 + 100 * 2.0**-15
    assert w[5].item() == 0.0
    # p is the nearest bf16 of w for every correction in the open half-spacing (away from a power of two, where the
    # spacing below is half as wide and the optimizer never produces a correction beyond -64)
    inside = torch.tensor([1.5] * 255, dtype=torch.bfloat16)
    cs = torch.arange(-127, 128, dtype=torch.int8)
    assert torch.equal(master_weight(inside, cs).bfloat16(), inside)


def _run(opt_name, steps, lr, seed=0, n=5000, wd=0.0):
    from halo_b200.optim.adamw_q8 import AdamWQ8, dequantize_moments, master_weight

    torch.manual_seed(seed)
    target = torch.randn(n)
    w0 = torch.randn(n) * 0.5
    if opt_name == "q8":
        p = torch.nn.Parameter(w0.bfloat16())
        opt = AdamWQ8([("w", p)], lr=lr, weight_decay=wd)
    else:
        p = torch.nn.Parameter(w0.bfloat16().float())
        opt = torch.optim.AdamW([p], lr=lr, weight_decay=wd)
    g = torch.Generator().manual_seed(seed + 1)
    for _ in range(steps):
        noise = torch.randn(n, generator=g) * 0.1
        grad = (p.detach().float() - target) + noise          # a noisy quadratic
        p.grad = grad.to(p.dtype)
        opt.step()
    if opt_name == "q8":
        st = opt.state[p]
        m, v = dequantize_moments(st["exp_avg_q"], st["exp_avg_sq_q"], st["exp_avg_scale"], st["exp_avg_sq_scale"])
        return master_weight(p, st["corr"]), m, v, opt
    st = opt.state[p]
    return p.detach().clone(), st["exp_avg"], st["exp_avg_sq"], opt


def test_long_run_tracks_fp32_adamw_and_small_updates_accumulate():
    w_q, m_q, v_q, opt = _run("q8", 300, 1e-2)
    w_f, m_f, v_f, _ = _run("fp32", 300, 1e-2)
    assert opt.state_bytes_per_param() < 5.1
    rel = ((w_q - w_f).norm() / w_f.norm()).item()
    assert rel < 2e-2, rel
    assert ((v_q - v_f).norm() / v_f.norm()).item() < 0.1
    # a learning rate whose per-step update is far below bf16's spacing at 1.0 (2^-7): a bf16 weight with nearest rounding
    # would never move; the 24-bit weight follows fp32 AdamW
    w_q, _, _, _ = _run("q8", 200, 2e-5)
    w_f, _, _, _ = _run("fp32", 200, 2e-5)
    torch.manual_seed(0)
    torch.randn(5000)
    w0 = (torch.randn(5000) * 0.5).bfloat16().float()
    moved_f = (w_f - w0).norm().item()
    assert moved_f > 0
    assert ((w_q - w0) - (w_f - w0)).norm().item() < 0.1 * moved_f


def test_second_moment_decays_instead_of_sticking_to_its_grid_point():
    from halo_b200.optim.adamw_q8 import AdamWQ8, dequantize_moments

    p = torch.nn.Parameter(torch.ones(512, dtype=torch.bfloat16))
    opt = AdamWQ8([("w", p)], lr=0.0, betas=(0.9, 0.99))
    p.grad = torch.ones(512, dtype=torch.bfloat16)
    opt.step()
    st = opt.state[p]
    _, v1 = dequantize_moments(st["exp_avg_q"], st["exp_avg_sq_q"], st["exp_avg_scale"], st["exp_avg_sq_scale"])
    for _ in range(200):
        p.grad = torch.zeros(512, dtype=torch.bfloat16)
        opt.step()
    _, v2 = dequantize_moments(st["exp_avg_q"], st["exp_avg_sq_q"], st["exp_avg_scale"], st["exp_avg_sq_scale"])
    want = v1.mean().item() * 0.99**200
    assert abs(v2.mean().item() / want - 1) < 0.05
    assert int(st["exp_avg_sq_q"].min()) >= 1          # a positive second moment never gets code 0


def test_same_names_same_noise_and_resume_is_exact():
    import copy

    from halo_b200.optim.adamw_q8 import AdamWQ8

    def make():
        torch.manual_seed(3)
        p = torch.nn.Parameter(torch.randn(40, 33).bfloat16())
        q = torch.nn.Parameter(torch.randn(33))            # an fp32 norm takes the plain path
        return p, q, AdamWQ8([("a.weight", p), ("a.norm", q)], lr=1e-2)

    def grads(p, q, i):
        g = torch.Generator().manual_seed(100 + i)
        p.grad = torch.randn(p.shape, generator=g).bfloat16()
        q.grad = torch.randn(q.shape, generator=g)

    p1, q1, o1 = make()
    for i in range(6):
        grads(p1, q1, i)
        o1.step()
    p2, q2, o2 = make()
    for i in range(3):
        grads(p2, q2, i)
        o2.step()
    saved = copy.deepcopy(o2.state_dict())
    weights = (p2.detach().clone(), q2.detach().clone())
    p3, q3, o3 = make()
    with torch.no_grad():
        p3.copy_(weights[0]), q3.copy_(weights[1])
    o3.load_state_dict(saved)
    for i in range(3, 6):
        grads(p3, q3, i)
        o3.step()
    assert torch.equal(p1, p3) and torch.equal(q1, q3)
    assert torch.equal(o1.state[p1]["corr"], o3.state[p3]["corr"])
    assert torch.equal(o1.state[p1]["exp_avg_sq_q"], o3.state[p3]["exp_avg_sq_q"])
    # a skip flag and a clip coefficient are honoured
    before = p1.detach().clone()
    grads(p1, q1, 9)
    o1.arm_skip(torch.ones(1, dtype=torch.int32))
    o1.step()
    assert torch.equal(p1, before)


def test_factory_builds_it_under_both_names():
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.optim.adamw_q8 import AdamWQ8
    from halo_b200.optim.factory import build_optimizer

    model = build_model(PRESETS["tiny-moe"](), device="cpu", dtype=torch.bfloat16)
    for name in ("adamw_q8", "flash_adamw"):
        assert isinstance(build_optimizer(model, name, lr=1e-4), AdamWQ8)
