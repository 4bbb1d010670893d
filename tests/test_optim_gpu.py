"""AdamWBF16 CUDA step against its bit-exact CPU twin, and the device-side clip / skip hand-off."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(n_list, seed=0):
    g = torch.Generator().manual_seed(seed)
    ps = [(f"layer.{i}.w", torch.randn(n, generator=g).bfloat16()) for i, n in enumerate(n_list)]
    gs = [torch.randn(n, generator=g).bfloat16() * 0.01 for n in n_list]
    return ps, gs


@pytest.mark.parametrize("grad_dtype", [torch.bfloat16, torch.float32])
def test_adamw_bf16_bit_exact(grad_dtype):
    from halo_b200.optim.adamw_bf16 import AdamWBF16

    sizes = [1, 7, 1024, 16384, 16385, 100003]
    ps, gs = _make(sizes)
    cpu = [(n, torch.nn.Parameter(p.clone())) for n, p in ps]
    gpu = [(n, torch.nn.Parameter(p.clone().cuda())) for n, p in ps]
    oc = AdamWBF16(cpu, lr=1e-3, weight_decay=0.01)
    og = AdamWBF16(gpu, lr=1e-3, weight_decay=0.01)
    for step in range(3):
        for (_, pc), (_, pg), g in zip(cpu, gpu, gs):
            gg = (g * (step + 1)).to(grad_dtype)
            if grad_dtype != pc.dtype:
                pc.grad_dtype = grad_dtype
                pg.grad_dtype = grad_dtype
            pc.grad = gg.clone()
            pg.grad = gg.clone().cuda()
        scale = torch.tensor([0.37])
        oc.defer_grad_scale(scale)
        og.defer_grad_scale(scale.cuda())
        oc.step()
        og.step()
        for (n, pc), (_, pg) in zip(cpu, gpu):
            assert torch.equal(pc.data, pg.data.cpu()), f"param {n} differs at step {step}"
            assert torch.equal(oc.state[pc]["exp_avg"], og.state[pg]["exp_avg"].cpu())
            assert torch.equal(oc.state[pc]["exp_avg_sq"], og.state[pg]["exp_avg_sq"].cpu())


def test_skip_flag_and_grad_norm():
    from halo_b200.optim.adamw_bf16 import AdamWBF16, GradNorm

    ps, gs = _make([5000, 33333], seed=3)
    gpu = [(n, torch.nn.Parameter(p.clone().cuda())) for n, p in ps]
    opt = AdamWBF16(gpu, lr=1e-2)
    for (_, p), g in zip(gpu, gs):
        p.grad = g.cuda()
    gn = GradNorm("cuda")
    gn.accumulate([p.grad for _, p in gpu])
    gn.finish(1.0)
    ref = torch.sqrt(sum(g.float().pow(2).sum() for g in gs))
    assert abs(gn.norm.item() - ref.item()) <= 1e-3 * ref.item()
    assert gn.skip.item() == 0
    assert abs(gn.coef.item() - min(1.0, 1.0 / (ref.item() + 1e-6))) < 1e-5
    before = [p.detach().clone() for _, p in gpu]
    gpu[0][1].grad[0] = float("nan")
    gn.accumulate([p.grad for _, p in gpu])
    gn.finish(1.0)
    assert gn.skip.item() == 1
    opt.defer_grad_scale(gn.coef)
    opt.arm_skip(gn.skip)
    opt.step()
    for b, (_, p) in zip(before, gpu):
        assert torch.equal(b, p.detach())


@pytest.mark.parametrize("host_compute", [False, True])
def test_host_state_optimizer_matches_the_device_optimizer_bit_for_bit(host_compute):
    """Moments in host memory - streamed through the device, or updated on the host CPU - give the very weights
    and moments of the all-device optimizer after several clipped steps."""
    from halo_b200.optim.adamw_bf16 import AdamWBF16, GradNorm
    from halo_b200.optim.offload import HostStateAdamWBF16

    torch.manual_seed(0)
    shapes = {"a.big": (300, 1000), "b.small": (17, 33), "c.big": (128, 4096)}
    base = {n: torch.randn(s, device="cuda").bfloat16() for n, s in shapes.items()}
    ref_p = [(n, torch.nn.Parameter(t.clone())) for n, t in base.items()]
    off_p = [(n, torch.nn.Parameter(t.clone())) for n, t in base.items()]
    ref = AdamWBF16(ref_p, lr=1e-2, weight_decay=0.1)
    off = HostStateAdamWBF16(off_p, lr=1e-2, weight_decay=0.1, host_min_numel=100_000, host_compute=host_compute)
    norm_r, norm_o = GradNorm(torch.device("cuda")), GradNorm(torch.device("cuda"))
    for step in range(4):
        g = {n: (torch.randn(s, device="cuda") * (3.0 if step == 2 else 0.3)).bfloat16() for n, s in shapes.items()}
        for params, opt, norm in ((ref_p, ref, norm_r), (off_p, off, norm_o)):
            for n, p in params:
                p.grad = g[n].clone()
            norm.accumulate([p.grad for _, p in params], first=True)
            norm.finish(1.0)
            opt.defer_grad_scale(norm.coef)
            opt.arm_skip(norm.skip)
            opt.step()
            opt.zero_grad(set_to_none=True)
        off.wait_all_ready()
        torch.cuda.synchronize()
    off.synchronize_state()
    assert off.state_bytes_on_host() > 0
    for (n, a), (_, b) in zip(ref_p, off_p):
        assert torch.equal(a.detach().view(torch.int16), b.detach().view(torch.int16)), n
        sa, sb = ref.state[a], off.state[b]
        for key in ("exp_avg", "exp_avg_sq"):        # host-resident moments are kept flat
            assert torch.equal(sa[key].cpu().reshape(-1).view(torch.int16), sb[key].cpu().reshape(-1).view(torch.int16)), (n, key)


@pytest.mark.parametrize("grad_dtype", [torch.bfloat16, torch.float32])
def test_adamw_q8_kernel_equals_its_tensor_op_statement(grad_dtype):
    """8-bit moments and 24-bit weights: the CUDA step against the CPU twin, bit for bit, over several steps (tensors whose
    length is not a multiple of the group, of a lane's eight elements, or of a block; one whose storage is offset so that
    the vector path is refused)."""
    from halo_b200.optim.adamw_q8 import AdamWQ8

    sizes = [1, 7, 256, 1000, 2048, 2049, 16385, 100003]
    ps, gs = _make(sizes, seed=5)
    cpu = [(n, torch.nn.Parameter(p.clone())) for n, p in ps]
    gpu = [(n, torch.nn.Parameter(p.clone().cuda())) for n, p in ps]
    # an unaligned view: the parameter starts 2 bytes into its storage
    base = torch.randn(4097).bfloat16()
    cpu.append(("offset.w", torch.nn.Parameter(base.clone()[1:])))
    gpu.append(("offset.w", torch.nn.Parameter(base.clone().cuda()[1:])))
    gs.append(torch.randn(4096).bfloat16() * 0.01)
    oc = AdamWQ8(cpu, lr=1e-3, weight_decay=0.01)
    og = AdamWQ8(gpu, lr=1e-3, weight_decay=0.01)
    for step in range(4):
        for (_, pc), (_, pg), g in zip(cpu, gpu, gs):
            gg = (g * (step + 1)).to(grad_dtype)
            if grad_dtype != pc.dtype:
                pc.grad_dtype = grad_dtype
                pg.grad_dtype = grad_dtype
            pc.grad = gg.clone()
            pg.grad = gg.clone().cuda()
        scale = torch.tensor([0.37])
        oc.defer_grad_scale(scale)
        og.defer_grad_scale(scale.cuda())
        oc.step()
        og.step()
        for (n, pc), (_, pg) in zip(cpu, gpu):
            sc, sg = oc.state[pc], og.state[pg]
            assert torch.equal(pc.data, pg.data.cpu()), f"param {n} differs at step {step}"
            for key in ("corr", "exp_avg_q", "exp_avg_sq_q", "exp_avg_scale", "exp_avg_sq_scale"):
                assert torch.equal(sc[key], sg[key].cpu()), f"{key} of {n} differs at step {step}"
    skip = torch.ones(1, dtype=torch.int32, device="cuda")
    before = [pg.detach().clone() for _, pg in gpu]
    for (_, pg), g in zip(gpu, gs):
        pg.grad = g.to(grad_dtype).cuda()
    og.arm_skip(skip)
    og.step()
    assert all(torch.equal(a, pg) for a, (_, pg) in zip(before, gpu))
