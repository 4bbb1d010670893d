"""Kernels of the model families beyond the flagship (residual-stream ops, per-stream norm, gated mean,
masked-softmax backward, standalone SwiGLU, block-scaled fake quantisation) against fp32 PyTorch statements of the
same ops."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _compare(op, ref, inputs, bf16_mask, tol=3e-2):
    """Run ``op`` on bf16 CUDA copies (where ``bf16_mask`` says so) and ``ref`` on fp32 copies; compare outputs and
    every input gradient in relative max-norm."""
    dev = "cuda"
    a = [(x.to(dev).bfloat16() if m else x.to(dev)).requires_grad_(x.is_floating_point()) for x, m in zip(inputs, bf16_mask)]
    b = [(x.to(dev).bfloat16().float() if m else x.to(dev).float()).requires_grad_(True) for x, m in zip(inputs, bf16_mask)]
    ya, yb = op(*a), ref(*b)
    g = torch.randn(yb.shape, device=dev, generator=torch.Generator(device=dev).manual_seed(3))
    (ya.float() * g).sum().backward()
    (yb.float() * g).sum().backward()
    assert (ya.float() - yb.float()).abs().max() <= tol * yb.float().abs().max() + 1e-3
    for i, (p, q) in enumerate(zip(a, b)):
        assert p.grad is not None, i
        assert (p.grad.float() - q.grad).abs().max() <= tol * q.grad.abs().max() + 2e-3, i


@pytest.mark.parametrize("N", [1, 2, 4, 8])
@pytest.mark.parametrize("T,H", [(5, 64), (300, 2048)])
def test_stream_collapse_mix_inject(N, T, H):
    from halo_b200.ops import streams as S

    torch.manual_seed(N * 100 + T)
    stream, block = torch.randn(T, N, H), torch.randn(T, H)
    w, post, gate = torch.rand(T, N), torch.rand(T, N), torch.randn(T, N)
    comb = torch.softmax(torch.randn(T, N, N), dim=-1)
    _compare(S.collapse_streams, S.collapse_streams_reference, [stream, w], [True, False])
    _compare(S.mix_streams, S.mix_streams_reference, [block, stream, post, comb], [True, True, False, False])
    _compare(S.inject_streams, S.inject_streams_reference, [block, stream, gate], [True, True, False])


@pytest.mark.parametrize("N,iters", [(2, 1), (4, 20), (8, 4)])
def test_sinkhorn(N, iters):
    from halo_b200.ops import streams as S

    torch.manual_seed(N)
    comb = torch.softmax(torch.randn(777, N, N), dim=-1) + 1e-6
    _compare(lambda c: S.sinkhorn_knopp(c, iters, 1e-6), lambda c: S.sinkhorn_knopp_reference(c, iters, 1e-6), [comb], [False],
             tol=1e-4)
    with torch.no_grad():
        out = S.sinkhorn_knopp(comb.cuda(), iters, 1e-6)
    assert torch.allclose(out.cpu(), S.sinkhorn_knopp_reference(comb, iters, 1e-6), atol=1e-5)


def test_stream_projection():
    from halo_b200.ops import streams as S

    torch.manual_seed(0)
    T, N, H = 400, 4, 512
    stream, fn = torch.randn(T, N, H), torch.randn(N * N + 2 * N, N * H) * 0.05
    _compare(lambda s, f: S.project_streams(s, f, 1e-6), lambda s, f: S.project_streams_reference(s, f, 1e-6), [stream, fn],
             [True, False])


@pytest.mark.parametrize("streams", [1, 2, 4])
@pytest.mark.parametrize("rows,H", [(3, 64), (1100, 1024)])
def test_grouped_rms_norm_and_gate_mix(streams, rows, H):
    from halo_b200.ops import streams as S

    torch.manual_seed(streams + rows)
    x, w = torch.randn(rows, streams * H), torch.randn(streams * H) * 0.1
    _compare(lambda a, b: S.grouped_rms_norm(a, b, 1e-6, streams), lambda a, b: S.grouped_rms_norm_reference(a, b, 1e-6, streams),
             [x, w], [True, False])
    normed, down, w_up = torch.randn(rows, streams * H), torch.randn(rows, 16), torch.randn(streams * H, 16) * 0.3
    _compare(lambda a, b, c: S.gate_mix(a, b, c, streams), lambda a, b, c: S.gate_mix_reference(a, b, c, streams),
             [normed, down, w_up], [True, True, True], tol=5e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_masked_softmax_backward(dtype):
    from halo_b200.ops import streams as S

    torch.manual_seed(1)
    heads, Q, K, scale = 4, 70, 333, 0.2
    scores = torch.randn(heads, Q, K, device="cuda")
    allowed = torch.rand(Q, K, device="cuda") > 0.4
    allowed[:, 0] = True
    masked = (scores * scale).masked_fill(~allowed, float("-inf"))
    lse = torch.logsumexp(masked, dim=-1)
    upstream = torch.randn(heads, Q, K, device="cuda")
    probs = torch.softmax(masked, dim=-1)
    delta = (probs * upstream).sum(-1)
    want_d = probs * (upstream - delta.unsqueeze(-1)) * scale
    p, d = S.masked_softmax_backward(scores, allowed, lse, scale, upstream, delta, True, dtype)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert p.dtype == dtype and (p.float() - probs).abs().max() <= tol
    assert (d.float() - want_d).abs().max() <= tol * max(1.0, want_d.abs().max().item())
    # a strided mask view and the probabilities alone
    wide = torch.zeros(Q, K + 5, device="cuda", dtype=torch.bool)
    wide[:, :K] = allowed
    p2, none = S.masked_softmax_backward(scores, wide[:, :K], lse, scale, writes_probs=True, dtype=dtype)
    assert none is None and torch.equal(p2, p)


def test_standalone_swiglu():
    from halo_b200.ops.activation import swiglu, swiglu_reference

    torch.manual_seed(2)
    pre = torch.randn(513, 2 * 768)
    _compare(swiglu, swiglu_reference, [pre], [True])


@pytest.mark.parametrize("fmt", ["mxfp8", "mxfp4", "nvfp4"])
def test_fake_quant_kernel_is_bit_identical_to_the_tensor_ops(fmt):
    from halo_b200.ops import lowp

    torch.manual_seed(4)
    x = (torch.randn(257, 1024, device="cuda") * torch.logspace(-6, 3, 1024, device="cuda")).bfloat16()
    x[3, :32] = 0
    got = lowp.fake_quant(x, fmt)
    want = lowp.fake_quant_reference(x, fmt)
    assert got.dtype == x.dtype and torch.equal(got, want)


@pytest.mark.parametrize("heads,kv_heads,D", [(32, 4, 128), (8, 8, 128), (4, 2, 64), (16, 1, 128)])
def test_decode_attention_kernel(heads, kv_heads, D):
    from halo_b200.inference.generate import KVCache

    torch.manual_seed(heads + D)
    B, S, layers = 5, 300, 2
    cache = KVCache(layers, B, S, kv_heads, D, torch.bfloat16, "cuda")
    cache.k.copy_(torch.randn_like(cache.k.float()))
    cache.v.copy_(torch.randn_like(cache.v.float()))
    cache.lengths.copy_(torch.tensor([0, 1, 7, 131, 298], device="cuda"))        # one key up to nearly the whole cache
    cache.begin_decode()
    q = torch.randn(B, heads * D, device="cuda").bfloat16()
    got = cache.attend(1, q, heads)
    # the same cache read by the tensor-op path (fp32 copies are not bf16: that path does not dispatch to the kernel)
    ref = KVCache(layers, B, S, kv_heads, D, torch.float32, "cuda")
    ref.k.copy_(cache.k.float())
    ref.v.copy_(cache.v.float())
    ref.lengths.copy_(cache.lengths)
    ref.begin_decode()
    want = ref.attend(1, q.float(), heads)
    assert got.dtype == torch.bfloat16 and (got.float() - want).abs().max() <= 2e-2 * want.abs().max() + 2e-3


def test_generation_on_gpu_matches_teacher_forcing():
    """Greedy sampling through the cache (packed prefill on the flash kernel, decode kernel) against the full forward of
    the grown sequence at every step."""
    import numpy as np

    from halo_b200.data.packing import pack_documents
    from halo_b200.inference.generate import Generator, SamplingParams
    from halo_b200.models.config import ModelConfig
    from halo_b200.models.qwen3 import build_model

    cfg = ModelConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=128, intermediate_size=512, moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2)
    model = build_model(cfg, device="cuda", seed=3, gradient_checkpointing=False)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 512, size=n) for n in (9, 33, 17)]
    outs = Generator(model).generate(prompts, SamplingParams(max_new_tokens=5, temperature=0.0))
    agree = total = 0
    for p, g in zip(prompts, outs):
        seq = list(p)
        for tok in g.token_ids:
            b = pack_documents([np.asarray(seq)]).to("cuda")
            with torch.no_grad():
                h = model.hidden_states(b.input_ids, b.position_ids, b.cu_seqlens)
                logits = h[-1].float() @ model.head_weight().float().t()
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) > 0.05:        # bf16 noise may flip a near tie; clear winners must agree
                agree += int(int(logits.argmax()) == int(tok))
                total += 1
            seq.append(int(tok))
    assert total >= 5 and agree == total


@pytest.mark.parametrize("kind", ["nf4", "fp4"])
@pytest.mark.parametrize("nested", [False, True])
@pytest.mark.parametrize("shape", [(64, 64), (768, 2048), (3, 5, 128)])
def test_4bit_dequantisation_kernel_is_bit_identical_to_the_tensor_ops(kind, nested, shape):
    from halo_b200.ops.nf4 import dequantize_4bit, dequantize_4bit_reference, quantize_4bit

    w = (torch.randn(shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)) * 0.05).bfloat16()
    packed = quantize_4bit(w, kind, nested)
    got, want = dequantize_4bit(packed), dequantize_4bit_reference(packed)
    assert got.dtype == torch.bfloat16 and got.shape == w.shape
    assert torch.equal(got, want)
    assert (got.float() - w.float()).abs().max() <= 0.17 * w.float().abs().max()


def test_quantized_base_on_gpu_equals_the_rounded_model():
    """QLoRA on the GPU: with the base in 4 bits the loss and the adapter gradients are those of the same model holding the
    rounded matrices in bf16 (same kernels, same inputs: equal up to the order of atomics-free reductions, i.e. exactly)."""
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import ModelConfig
    from halo_b200.models.qwen3 import build_model
    from halo_b200.peft.lora import LoraSpec, apply_lora
    from halo_b200.peft.qlora import dequantized_base_state, quantize_base_weights

    cfg = ModelConfig(vocab_size=4096, hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=128, moe_intermediate_size=256, num_experts=8, num_experts_per_tok=2)
    batch = synthetic_packed_batch(512, cfg.vocab_size, seed=0, lo=64, hi=200).to("cuda")

    def make():
        m = build_model(cfg, device="cuda", seed=0)
        apply_lora(m, LoraSpec(r=8, alpha=16.0, target_modules=["q_proj", "v_proj", "o_proj"]), seed=0)
        with torch.no_grad():
            for n, p in m.named_parameters():
                if p.requires_grad and ".lora.B." in n:
                    p.normal_(0.0, 0.02)
        return m

    torch.manual_seed(0)
    q = make()
    torch.manual_seed(0)
    plain = make()
    quantize_base_weights(q, "nf4", nested=True)
    with torch.no_grad():
        for name, rounded in dequantized_base_state(q).items():
            plain.get_parameter(name).copy_(rounded)
    losses = []
    for m in (q, plain):
        out = m(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
        loss = out.loss if hasattr(out, "loss") else out
        loss.sum().backward()
        losses.append(loss.detach().float().sum())
    assert torch.isfinite(losses[0]) and abs(float(losses[0] - losses[1])) <= 1e-3 * abs(float(losses[1]))
    grads = {n: p.grad for n, p in plain.named_parameters() if p.requires_grad}
    for n, p in q.named_parameters():
        if p.requires_grad:
            assert p.grad is not None and torch.isfinite(p.grad).all(), n
            assert (p.grad.float() - grads[n].float()).abs().max() <= 2e-2 * grads[n].float().abs().max() + 1e-6, n


def _gpu_family_config(family):
    from halo_b200.models.config import FAMILIES, ModelConfig

    base = dict(vocab_size=2048, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                intermediate_size=512, moe_intermediate_size=0, num_experts=0, model_type=family, rope_theta=10000.0,
                max_position_embeddings=4096, use_qk_norm=FAMILIES[family]["qk_norm"], attention_bias=FAMILIES[family]["bias_default"])
    if FAMILIES[family]["moe"]:
        base.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, intermediate_size=256)
    extra = {
        "llama": dict(head_dim=128, num_attention_heads=2, num_key_value_heads=1),
        "mistral": dict(sliding_window=64),
        "gpt_oss": dict(sliding_window=64, layer_types=["sliding_attention", "full_attention"], attention_sinks=True, output_bias=True,
                        router_logit_bias=True, expert_bias=True, expert_activation="clamped_glu", rms_norm_eps=1e-5),
        "deepseek_v3": dict(score_function="sigmoid", router_bias=True, n_group=2, topk_group=1, routed_scaling_factor=2.5,
                            shared_expert_intermediate_size=256, mlp_only_layers=[0], use_qk_norm=False, num_key_value_heads=4,
                            intermediate_size=512, kv_lora_rank=64, q_lora_rank=96, qk_nope_head_dim=64, qk_rope_head_dim=64, v_head_dim=64),
        "gemma2": dict(sliding_window=64, layer_types=["sliding_attention", "full_attention"], use_qk_norm=False, hidden_activation="gelu_tanh",
                       sandwich_norms=True, norm_unit_offset=True, embedding_multiplier=16.0, query_pre_attn_scalar=96,
                       attn_logit_softcapping=20.0, final_logit_softcapping=10.0, tie_word_embeddings=True),
        "gemma3_text": dict(sliding_window=64, layer_types=["sliding_attention", "full_attention"], hidden_activation="gelu_tanh",
                            sandwich_norms=True, norm_unit_offset=True, embedding_multiplier=16.0, query_pre_attn_scalar=96,
                            rope_local_theta=500.0, tie_word_embeddings=True),
    }[family]
    base.update(extra)
    return ModelConfig(**base)


@pytest.mark.parametrize("family", ["llama", "mistral", "gpt_oss", "deepseek_v3", "gemma2", "gemma3_text"])
def test_family_on_gpu_follows_its_fp32_cpu_twin(family):
    """The same weights in bf16 on the GPU and in fp32 on the CPU: loss within bf16 tolerance, finite gradients of matching
    size for every parameter (the family switches reach the same ops on both devices)."""
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.qwen3 import build_model

    cfg = _gpu_family_config(family)
    cpu = build_model(cfg, device="cpu", dtype=torch.float32, seed=3, gradient_checkpointing=False)
    gpu = build_model(cfg, device="cuda", seed=3)
    with torch.no_grad():
        for (n, a), (_, b) in zip(cpu.named_parameters(), gpu.named_parameters()):
            a.copy_(b.float())                                   # the bf16 values, exactly
    batch = synthetic_packed_batch(256, cfg.vocab_size, seed=0, lo=40, hi=130)
    losses, norms = [], []
    for model, b in ((cpu, batch), (gpu, batch.to("cuda"))):
        out = model(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
        loss = (out.loss if hasattr(out, "loss") else out).sum()
        loss.backward()
        losses.append(float(loss))
        grads = [p.grad for p in model.parameters() if p.requires_grad]
        assert all(g is not None and torch.isfinite(g).all() for g in grads), family
        norms.append(float(torch.sqrt(sum(g.float().pow(2).sum() for g in grads))))
    assert abs(losses[0] - losses[1]) <= 3e-2 * abs(losses[0]), (family, losses)
    assert abs(norms[0] - norms[1]) <= 0.15 * norms[0], (family, norms)
