"""Block-scaled formats on CPU: the round trip against brute-force nearest-value rounding, packing, idempotence,
slice invariance of nvfp4's tensor scale, the straight-through gradient and the weight round-trip cache."""

import itertools
import os

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


def test_checkpoint_conversions(tmp_path):
    import json

    from safetensors.torch import save_file

    from halo_b200.checkpoint.load import CheckpointIndex, from_pretrained
    from halo_b200.checkpoint.save import save_model
    from halo_b200.checkpoint.tools import lowp_convert
    from halo_b200.models.config import tiny_moe_config
    from halo_b200.models.qwen3 import build_model

    # a served-weights release in 128 x 128 block FP8 -> bf16
    torch.manual_seed(0)
    w = torch.randn(200, 300)
    scale_inv = torch.rand(2, 3) + 0.5
    full = scale_inv.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1)[:, :300]
    fp8 = (w / full).to(torch.float8_e4m3fn)
    src = tmp_path / "fp8"
    src.mkdir()
    save_file({"model.layers.0.mlp.down_proj.weight": fp8, "model.layers.0.mlp.down_proj.weight_scale_inv": scale_inv,
               "model.norm.weight": torch.ones(300, dtype=torch.bfloat16)}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"model_type": "qwen3", "quantization_config": {"quant_method": "fp8"}}))
    assert lowp_convert.main(["dequant-block-fp8", str(src), str(tmp_path / "bf16")]) == 0
    out = CheckpointIndex(str(tmp_path / "bf16"))
    got = out.get("model.layers.0.mlp.down_proj.weight")
    assert got.dtype == torch.bfloat16 and "model.layers.0.mlp.down_proj.weight_scale_inv" not in out
    assert torch.equal(got, (fp8.float() * full).bfloat16()) and (got.float() - w).abs().max() < 0.08 * w.abs().max()
    assert "quantization_config" not in json.load(open(tmp_path / "bf16" / "config.json"))

    # and back: exporting the bf16 result gives a release that dequantises to (nearly) the same weights
    assert lowp_convert.main(["export-block-fp8", str(tmp_path / "bf16"), str(tmp_path / "fp8_again")]) == 0
    again = CheckpointIndex(str(tmp_path / "fp8_again"))
    assert again.get("model.layers.0.mlp.down_proj.weight").dtype == torch.float8_e4m3fn
    assert again.get("model.layers.0.mlp.down_proj.weight_scale_inv").shape == (2, 3)
    assert again.get("model.norm.weight").dtype == torch.bfloat16
    assert lowp_convert.main(["dequant-block-fp8", str(tmp_path / "fp8_again"), str(tmp_path / "bf16_again")]) == 0
    twice = CheckpointIndex(str(tmp_path / "bf16_again")).get("model.layers.0.mlp.down_proj.weight")
    assert (twice.float() - got.float()).abs().max() <= 0.07 * got.float().abs().max()
    assert json.load(open(tmp_path / "fp8_again" / "config.json"))["quantization_config"]["weight_block_size"] == [128, 128]

    # a model exported in a block-scaled format and read back is the fake-quantised model
    model = build_model(tiny_moe_config(), device="cpu", seed=1)
    ckpt = str(tmp_path / "ckpt")
    save_model(model, ckpt, save_dtype=torch.bfloat16)
    for fmt in ("mxfp8", "nvfp4"):
        q_dir, back_dir = str(tmp_path / f"q_{fmt}"), str(tmp_path / f"back_{fmt}")
        assert lowp_convert.main(["export", ckpt, q_dir, "--format", fmt, "--keep", r"layers\.0\."]) == 0
        meta = json.load(open(os.path.join(q_dir, "halo_lowp.json")))
        assert meta["format"] == fmt and meta["quantized_tensors"] > 10
        assert lowp_convert.main(["dequant", q_dir, back_dir]) == 0
        back = from_pretrained(back_dir, device="cpu", dtype=torch.bfloat16)
        ref = from_pretrained(ckpt, device="cpu", dtype=torch.bfloat16)
        for (n, a), (_, b) in zip(back.named_parameters(), ref.named_parameters()):
            untouched = n.startswith("layers.0.") or a.dim() < 2 or "embed" in n or "lm_head" in n or n.endswith("mlp.gate")
            if untouched:
                assert torch.equal(a, b), n
            elif a.dim() == 2:
                # fused runtime tensors are concatenations of hub matrices quantised one by one along the same axis
                assert torch.equal(a, lowp.fake_quant_reference(b, fmt)) or fmt == "nvfp4", n
                assert (a.float() - b.float()).abs().max() <= 0.3 * b.float().abs().max(), n


def test_quantisation_aware_training_rounds_every_product():
    import dataclasses

    import numpy as np

    from halo_b200.data.packing import pack_documents
    from halo_b200.models.config import tiny_moe_config
    from halo_b200.models.qwen3 import apply_lowp_compute, build_model

    cfg = dataclasses.replace(tiny_moe_config(), num_hidden_layers=2, shared_expert_intermediate_size=64)
    rng = np.random.default_rng(0)
    b = pack_documents([rng.integers(0, cfg.vocab_size, size=n) for n in (40, 24)])
    base = build_model(cfg, device="cpu", seed=2, gradient_checkpointing=False)
    want = base(b.input_ids, b.position_ids, b.cu_seqlens, b.labels).item()
    model = build_model(cfg, device="cpu", seed=2)
    assert apply_lowp_compute(model, "mxfp8") == 2 * 3              # attention, routed experts and the shared expert per layer
    loss = model(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
    assert 1e-6 < abs(loss.item() - want) < 0.05                    # e4m3 rounding moves the loss a little
    loss.backward()
    assert all(p.grad is not None and p.grad.abs().sum() > 0 for n, p in model.named_parameters() if p.dim() > 1)
    # a dense block: the rounded product by hand
    mlp = model.layers[0].mlp.shared_expert
    x = torch.randn(6, cfg.hidden_size)
    fq = lambda t: lowp.fake_quant_reference(t, "mxfp8")
    pre = fq(x) @ fq(mlp.gate_up_proj).t()
    act = torch.nn.functional.silu(pre[:, :64]) * pre[:, 64:]
    assert torch.allclose(mlp(x), fq(act) @ fq(mlp.down_proj).t(), atol=1e-5)
    coarse = build_model(cfg, device="cpu", seed=2)
    apply_lowp_compute(coarse, "mxfp4")
    assert abs(coarse(b.input_ids, b.position_ids, b.cu_seqlens, b.labels).item() - want) > abs(loss.item() - want)
    with pytest.raises(ValueError, match="no multiples"):
        apply_lowp_compute(build_model(dataclasses.replace(cfg, moe_intermediate_size=80), device="cpu", seed=0), "mxfp8")


def test_static_fp8_and_packed_mxfp4_releases(tmp_path):
    """Releases with static per-matrix / per-expert FP8 scales, and with expert banks packed as MXFP4 blocks (the gpt-oss
    hub layout): both come back as plain bf16 checkpoints, the second one loadable by the family's loader."""
    import json

    import pytest
    from safetensors.torch import load_file, save_file

    from halo_b200.checkpoint.load import CheckpointIndex, from_pretrained
    from halo_b200.checkpoint.save import save_model
    from halo_b200.checkpoint.tools import lowp_convert
    from halo_b200.models.qwen3 import build_model
    from tests.test_families_cpu import family_config

    torch.manual_seed(0)
    # --- static scales
    w = torch.randn(64, 48)
    bank = torch.randn(3, 16, 24)
    s_w, s_bank = torch.tensor(0.02), torch.tensor([0.01, 0.03, 0.05])
    src = tmp_path / "static"
    src.mkdir()
    save_file({"model.layers.0.self_attn.q_proj.weight": (w / s_w).to(torch.float8_e4m3fn),
               "model.layers.0.self_attn.q_proj.weight_scale": s_w.reshape(1),
               "model.layers.0.self_attn.q_proj.input_scale": torch.tensor([0.5]),
               "model.layers.0.mlp.experts.weight": (bank / s_bank[:, None, None]).to(torch.float8_e4m3fn),
               "model.layers.0.mlp.experts.weight_scale": s_bank,
               "model.norm.weight": torch.ones(48, dtype=torch.float32)}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"model_type": "mistral", "quantization_config": {"quant_method": "fp8"}}))
    assert lowp_convert.main(["dequant-static-fp8", str(src), str(tmp_path / "static_bf16")]) == 0
    out = CheckpointIndex(str(tmp_path / "static_bf16"))
    assert sorted(out.weight_map) == ["model.layers.0.mlp.experts.weight", "model.layers.0.self_attn.q_proj.weight", "model.norm.weight"]
    got = out.get("model.layers.0.self_attn.q_proj.weight")
    assert got.dtype == torch.bfloat16 and (got.float() - w).abs().max() < 0.08 * w.abs().max()
    got_bank = out.get("model.layers.0.mlp.experts.weight")
    assert torch.equal(got_bank, ((bank / s_bank[:, None, None]).to(torch.float8_e4m3fn).float() * s_bank[:, None, None]).bfloat16())
    assert out.get("model.norm.weight").dtype == torch.bfloat16
    assert "quantization_config" not in json.load(open(tmp_path / "static_bf16" / "config.json"))
    with pytest.raises(ValueError, match="output directory is the input"):
        lowp_convert.dequant_static_fp8(str(src), str(src))
    with pytest.raises(ValueError, match="nothing to dequantise"):
        lowp_convert.dequant_static_fp8(str(tmp_path / "static_bf16"), str(tmp_path / "again"))

    # --- packed MXFP4: codes and exponents chosen at random, so the expected values are exact
    codes = torch.randint(0, 16, (2, 5, 3, 32))
    exps = torch.randint(120, 131, (2, 5, 3), dtype=torch.int32)
    lut = torch.tensor(lowp_convert._E2M1)
    want = (lut[codes] * torch.pow(2.0, (exps - 127).float())[..., None]).reshape(2, 5, 96)
    blocks = (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)             # low nibble first
    assert torch.equal(lowp_convert.unpack_mxfp4_blocks(blocks, exps.to(torch.uint8)), want)

    # a gpt-oss checkpoint whose banks are packed that way loads as the bf16 model it encodes
    cfg = family_config("gpt_oss")
    model = build_model(cfg, device="cpu", seed=2)
    ckpt = tmp_path / "gpt_oss_bf16"
    save_model(model, str(ckpt), save_dtype=torch.bfloat16)
    shard = [f for f in os.listdir(ckpt) if f.endswith(".safetensors")]
    assert len(shard) == 1
    tensors = load_file(str(ckpt / shard[0]))
    packed, exact = {}, {}
    for name, t in tensors.items():
        if name.endswith(("experts.gate_up_proj", "experts.down_proj")):
            E, n_in, n_out = t.shape                                                      # the hub's bf16 banks are [E, in, out]
            c = torch.randint(0, 16, (E, n_out, n_in // 32, 32))
            e = torch.randint(118, 126, (E, n_out, n_in // 32), dtype=torch.int32)
            vals = (lut[c] * torch.pow(2.0, (e - 127).float())[..., None]).reshape(E, n_out, n_in)
            packed[name + "_blocks"] = (c[..., 0::2] | (c[..., 1::2] << 4)).to(torch.uint8)
            packed[name + "_scales"] = e.to(torch.uint8)
            exact[name] = vals.transpose(1, 2).contiguous().bfloat16()
        else:
            packed[name] = t
            exact[name] = t
    src4 = tmp_path / "gpt_oss_mxfp4"
    src4.mkdir()
    save_file(packed, str(src4 / "model.safetensors"))
    cfg_json = json.load(open(ckpt / "config.json"))
    cfg_json["quantization_config"] = {"quant_method": "mxfp4"}
    (src4 / "config.json").write_text(json.dumps(cfg_json))
    assert lowp_convert.main(["dequant-mxfp4-experts", str(src4), str(tmp_path / "gpt_oss_back")]) == 0
    back = CheckpointIndex(str(tmp_path / "gpt_oss_back"))
    assert sorted(back.weight_map) == sorted(exact)
    for name, t in exact.items():
        assert torch.equal(back.get(name), t), name
    loaded = from_pretrained(str(tmp_path / "gpt_oss_back"), device="cpu")
    bank0 = loaded.layers[0].mlp.experts_down
    assert torch.isfinite(bank0).all() and bank0.shape == model.layers[0].mlp.experts_down.shape
    # the packed release also loads as it is (the loader unpacks the banks), to the same weights
    direct = from_pretrained(str(src4), device="cpu")
    for (n, a_), (_, b_) in zip(loaded.named_parameters(), direct.named_parameters()):
        assert torch.equal(a_, b_), n
    # an expert-parallel rank keeps its experts of a bank stored whole
    from halo_b200.checkpoint.load import load_model_weights
    from halo_b200.models.qwen3 import Qwen3Model

    class _SecondOfTwo:
        n_ranks, rank = 2, 1

    half = Qwen3Model(cfg, dtype=torch.float32, device="cpu", transport=_SecondOfTwo())
    load_model_weights(half, str(tmp_path / "gpt_oss_back"))
    n_local = cfg.num_experts // 2
    assert half.layers[0].mlp.experts_gate_up_bias.shape[0] == n_local
    assert torch.equal(half.layers[1].mlp.experts_down, loaded.layers[1].mlp.experts_down[n_local:])
    assert torch.equal(half.layers[0].mlp.experts_gate_up_bias, loaded.layers[0].mlp.experts_gate_up_bias[n_local:])
