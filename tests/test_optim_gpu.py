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
