"""tcgen05 GEMM against a plain fp32 PyTorch product, every operand layout and epilogue."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_t, b_t):
    af = a.float().t() if a_t else a.float()
    bf = b.float().t() if b_t else b.float()
    return af @ bf


def _rand(shape, scale=1.0):
    return (torch.randn(shape, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("a_t,b_t", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (256, 512, 256), (384, 264, 200), (1000, 776, 520), (4096, 2048, 1024)])
def test_matmul_layouts(a_t, b_t, mnk):
    from halo_b200.ops import _lib
    from halo_b200.ops.gemm import matmul

    M, N, K = mnk
    torch.manual_seed(0)
    a = _rand((K, M) if a_t else (M, K))
    b = _rand((N, K) if b_t else (K, N))
    out = matmul(a, b, a_t=a_t, b_t=b_t)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    ref = _ref(a, b, a_t, b_t)
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-3
    assert err <= tol, f"max err {err} > {tol}"


def test_matmul_fp32_and_accumulate():
    from halo_b200.ops.gemm import matmul

    torch.manual_seed(1)
    a, b = _rand((512, 320)), _rand((264, 320))
    ref = _ref(a, b, False, True)
    out = matmul(a, b, out_dtype=torch.float32)
    assert (out - ref).abs().max().item() <= 1e-3 * ref.abs().max().item() + 1e-4
    acc = torch.ones_like(out)
    matmul(a, b, out=acc, accumulate=True, alpha=0.5)
    assert (acc - (1 + 0.5 * ref)).abs().max().item() <= 1e-3 * ref.abs().max().item() + 1e-4
    accb = torch.ones((512, 264), dtype=torch.bfloat16, device="cuda")
    matmul(a, b, out=accb, accumulate=True)
    assert (accb.float() - (1 + ref)).abs().max().item() <= 2e-2 * ref.abs().max().item()


def test_swiglu_epilogue():
    from halo_b200.ops.gemm import swiglu_matmul

    torch.manual_seed(2)
    x, w = _rand((777, 512)), _rand((2 * 384, 512), 0.05)
    act, pre = swiglu_matmul(x, w, save_pre=True)
    pre_ref = (x.float() @ w.float().t())
    assert (pre.float() - pre_ref).abs().max().item() <= 2e-2 * pre_ref.abs().max().item()
    g, u = pre.float()[:, :384], pre.float()[:, 384:]
    act_ref = torch.nn.functional.silu(g) * u
    assert (act.float() - act_ref).abs().max().item() <= 1e-2 * act_ref.abs().max().item() + 1e-3


def test_linear_autograd():
    from halo_b200.ops.gemm import linear

    torch.manual_seed(3)
    x = _rand((3, 100, 256)).requires_grad_()
    w = _rand((384, 256), 0.05).requires_grad_()
    y = linear(x, w)
    gy = _rand(y.shape)
    y.backward(gy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(gy.float())
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad)):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3


@pytest.mark.parametrize("a_t,b_t", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("mnk", [(2048, 1024, 2048), (1000, 520, 1600), (304, 2048, 4096)])
def test_pair_kernel_shapes(a_t, b_t, mnk):
    """Long reductions with narrow outputs take the CTA-pair (cta_group::2) kernel; odd sizes exercise the half
    tiles of the second CTA and the clipped edges."""
    from halo_b200.ops import _lib
    from halo_b200.ops.gemm import matmul

    M, N, K = mnk
    torch.manual_seed(1)
    a = _rand((K, M) if a_t else (M, K), 0.3)
    b = _rand((N, K) if b_t else (K, N), 0.3)
    out = matmul(a, b, a_t=a_t, b_t=b_t)
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    ref = _ref(a, b, a_t, b_t)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err


def test_every_product_on_the_pair_kernel_in_a_fresh_process():
    """HALO_GEMM_PAIR=2 routes every dense and grouped product through the pair kernel; the kernel choice is read
    once per process, so the GEMM and MoE numerics run again in a child process with the switch set."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, HALO_GEMM_PAIR="2")
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gemm_gpu.py", "tests/test_moe_gpu.py", "-q", "-m", "gpu", "-x",
                        "-k", "not fresh_process"], cwd=root, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
