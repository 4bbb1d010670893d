"""Block-scaled formats on CPU: the round trip against brute-force nearest-value rounding, packing, idempotence,
slice invariance of nvfp4's tensor scale, the straight-through gradient and the weight round-trip cache."""

import itertools

import pytest
import torch

from halo_b200.ops import lowp

LEVELS = torch.tensor(lowp._E2M1_LEVELS)


def brute_e2m1(x):
    """Nearest e2m1 magnitude, ties to the even code, by exhaustive comparison in float64."""
    mag = x.abs().double().clamp(max=6.0)
    d = (mag.unsqueeze(-1) - LEVELS.double()).abs()
    best = d.min(-1).values
    codes = torch.arange(8)
    is_best = d == best.unsqueeze(-1)
    even_first = torch.where(is_best & (codes % 2 == 0), 0, torch.where(is_best, 1, 2))
    pick = even_first.argmin(-1)
    return torch.where(x < 0, -LEVELS[pick], LEVELS[pick])


def test_e2m1_rounding_is_nearest_with_ties_to_even():
    grid = torch.linspace(-7, 7, 1121)        # step 1/80: hits every midpoint exactly
    got = lowp._e2m1_values(lowp._e2m1_codes(grid))
    assert torch.equal(got, brute_e2m1(grid).float())
    assert lowp._e2m1_values(lowp._e2m1_codes(torch.tensor([0.75, 0.25, 2.5, 3.5, 5.0, 1.25, 1.75]))).tolist() == [1.0, 0.0, 2.0, 4.0, 4.0, 1.0, 2.0]


@pytest.mark.parametrize("fmt", lowp.FORMATS)
def test_round_trip_properties(fmt):
    torch.manual_seed(0)
    # nine decades for the MX formats; two for nvfp4, whose e4m3 block scale spans ~4.6 decades below the tensor's max
    x = (torch.randn(64, 256) * (torch.logspace(-5, 4, 256) if fmt != "nvfp4" else torch.logspace(-2, 0, 256))).bfloat16()
    x[5, :32] = 0
    y = lowp.fake_quant(x, fmt)
    assert y.dtype == x.dtype and y.shape == x.shape
    assert torch.equal(lowp.fake_quant(y, fmt), y) or fmt == "nvfp4"       # MX: a representable tensor stays put
    assert torch.equal(y[5, :32], torch.zeros(32, dtype=x.dtype))
    q = lowp.quantize(x, fmt)
    bs = lowp.BLOCK_SIZE[fmt]
    assert q.scales.shape == (64, 256 // bs)
    assert q.data.shape == ((64, 256) if fmt == "mxfp8" else (64, 128))
    assert torch.equal(lowp.dequantize(q, x.dtype), y)
    # the error of a block is bounded by half a step at the block's scale
    blocks, yb = x.float().view(64, -1, bs), y.float().view(64, -1, bs)
    amax = blocks.abs().amax(-1, keepdim=True)
    step = {"mxfp8": 2.0 ** -3, "mxfp4": 0.5, "nvfp4": 0.5}[fmt]     # relative spacing at the top binade / coarsest gap
    assert ((blocks - yb).abs() <= amax * step + 1e-30).all()


def test_mx_scale_is_the_smallest_power_of_two_that_fits():
    for fmt, amax in itertools.product(("mxfp8", "mxfp4"), (448.0, 449.0, 6.0, 6.5, 1.0, 3e-5, 2.0 ** -20)):
        x = torch.zeros(1, 32)
        x[0, 3] = amax
        q = lowp.quantize(x, fmt)
        e = int(q.scales[0, 0]) - 127
        top = lowp.ELEMENT_MAX[fmt]
        assert amax <= top * 2.0 ** e and amax > top * 2.0 ** (e - 1), (fmt, amax, e)


def test_nvfp4_slices_quantise_as_the_whole():
    torch.manual_seed(1)
    w = torch.randn(32, 128) * 0.02
    whole = lowp.quantize(w, "nvfp4")
    part = lowp.quantize(w[:16], "nvfp4", global_scale=whole.global_scale)
    assert torch.equal(part.data, whole.data[:16]) and torch.equal(part.scales.view(torch.uint8), whole.scales[:16].view(torch.uint8))
    gs = float(whole.global_scale)
    assert gs == 2.0 ** round(torch.log2(torch.tensor(gs)).item()) and float(w.abs().max()) <= gs * 448 * 6


def test_straight_through_gradient_and_linear():
    x = torch.randn(8, 64, requires_grad=True)
    w = torch.randn(16, 64, requires_grad=True)
    y = lowp.lowp_linear(x, w, "mxfp8")
    want = lowp.fake_quant_reference(x.detach(), "mxfp8") @ lowp.fake_quant_reference(w.detach(), "mxfp8").t()
    assert torch.allclose(y, want, atol=1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    assert torch.allclose(x.grad, g @ lowp.fake_quant_reference(w.detach(), "mxfp8"), atol=1e-5)
    assert torch.allclose(w.grad, g.t() @ lowp.fake_quant_reference(x.detach(), "mxfp8"), atol=1e-5)
    with pytest.raises(ValueError, match="not a multiple"):
        lowp.fake_quant(torch.randn(4, 40), "mxfp8")


def test_weight_cache_follows_in_place_updates():
    cache = lowp.WeightRoundTripCache()
    w = torch.randn(4, 32)
    a = cache.get(w, "mxfp4")
    assert cache.get(w, "mxfp4") is a
    w.add_(1.0)
    b = cache.get(w, "mxfp4")
    assert b is not a and torch.equal(b, lowp.fake_quant_reference(w, "mxfp4"))
