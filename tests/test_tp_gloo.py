"""Tensor parallelism with token-sharded activations on two gloo ranks: a dense and a MoE model give the loss
and the gradients of the unsliced model; weight slices reassemble to the full tensors."""

import pytest
import torch

from halo_b200.models.config import PRESETS, ModelConfig
from halo_b200.parallel.tensor_parallel import slice_for_rank, unslice
from tests.common.gloo import run_gloo_ranks


def test_slices_reassemble():
    cfg = ModelConfig(hidden_size=64, num_attention_heads=8, num_key_value_heads=4, head_dim=16, intermediate_size=96)
    shapes = {"qkv": (cfg.qkv_dim, 64), "o": (64, 8 * 16), "gate_up": (2 * 96, 64), "down": (64, 96)}
    for kind, shape in shapes.items():
        full = torch.randn(shape)
        for size in (2, 4):
            parts = [slice_for_rank(kind, full, cfg, r, size) for r in range(size)]
            assert torch.equal(unslice(kind, parts, cfg), full), (kind, size)


def _worker(rank, world, preset):
    import dataclasses

    import numpy as np
    import torch.distributed as dist

    from halo_b200.data.packing import PackedBatch, pack_documents
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.tensor_parallel import TensorParallel, gather_full_weight

    if preset == "dense":
        cfg = ModelConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                          head_dim=16, intermediate_size=96, num_experts=0, model_type="qwen3")
    else:
        cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2)
    rng = np.random.default_rng(1)
    full = pack_documents([rng.integers(0, cfg.vocab_size, size=n) for n in (50, 31, 47)])     # 128 tokens
    norm = float(full.n_scored)
    tp = TensorParallel(dist.group.WORLD, "cpu")
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=4, tensor_parallel=tp)
    lo, hi = tp.shard_rows(full.n_tokens)
    # token ids and labels are this rank's shard; positions and document boundaries describe the whole row
    ctx = model.make_context(full.position_ids, full.cu_seqlens)
    local = PackedBatch(full.input_ids[lo:hi], full.position_ids, full.labels[lo:hi], full.cu_seqlens, 0)
    loss = model(local.input_ids, local.position_ids, local.cu_seqlens, local.labels, norm, ctx=ctx)
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)

    ref = build_model(cfg, device="cpu", dtype=torch.float32, seed=4)
    ref_loss = ref(full.input_ids, full.position_ids, full.cu_seqlens, full.labels, norm)
    ref_loss.backward()
    assert torch.allclose(total, ref_loss.detach(), rtol=1e-5, atol=1e-6), (float(total), float(ref_loss))
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        kind = getattr(p, "tp_kind", None)
        if kind is None:
            g = p.grad.clone()
            dist.all_reduce(g)                       # replicated weights saw only this rank's tokens
            want_w, want_g = ref_params[name].detach(), ref_params[name].grad
        else:
            g = gather_full_weight(kind, p.grad, cfg, tp)          # sliced weights saw every token
            want_w, want_g = ref_params[name].detach(), ref_params[name].grad
            assert torch.equal(gather_full_weight(kind, p.detach(), cfg, tp), want_w), name
        assert torch.allclose(g, want_g, rtol=2e-4, atol=2e-6), name


@pytest.mark.parametrize("preset", ["dense", "moe"])
def test_tensor_parallel_matches_unsliced_model(preset):
    run_gloo_ranks(_worker, 2, args=(preset,), timeout=120.0)


def _etp_worker(rank, world):
    import dataclasses

    import numpy as np
    import torch.distributed as dist

    from halo_b200.data.packing import pack_documents
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.expert_tensor_parallel import ExpertTensorParallel, unslice_expert_bank

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2)
    rng = np.random.default_rng(2)
    batch = pack_documents([rng.integers(0, cfg.vocab_size, size=n) for n in (40, 70, 18)])
    etp = ExpertTensorParallel(dist.group.WORLD)
    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=6, expert_tensor_parallel=etp)
    loss = model(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)     # every rank: the same tokens
    loss.backward()
    ref = build_model(cfg, device="cpu", dtype=torch.float32, seed=6)
    ref_loss = ref(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
    ref_loss.backward()
    assert torch.allclose(loss.detach(), ref_loss.detach(), rtol=1e-5, atol=1e-6)
    ref_params = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        kind = getattr(p, "etp_kind", None)
        if kind is None:
            assert torch.allclose(p.grad, ref_params[name].grad, rtol=2e-4, atol=2e-6), name   # replicated: same on every rank
        else:
            parts = [torch.empty_like(p.grad) for _ in range(world)]
            dist.all_gather(parts, p.grad.contiguous())
            assert torch.allclose(unslice_expert_bank(kind, parts), ref_params[name].grad, rtol=2e-4, atol=2e-6), name
            wparts = [torch.empty_like(p.detach()) for _ in range(world)]
            dist.all_gather(wparts, p.detach().contiguous())
            assert torch.equal(unslice_expert_bank(kind, wparts), ref_params[name].detach()), name


def test_expert_tensor_parallel_matches_unsliced_experts():
    run_gloo_ranks(_etp_worker, 2, timeout=120.0)


def _sliced_load_worker(rank, world, directory):
    import torch.distributed as dist

    from halo_b200.checkpoint.load import from_pretrained
    from halo_b200.parallel.tensor_parallel import TensorParallel, gather_full_weight

    tp = TensorParallel(dist.group.WORLD, "cpu")
    whole = from_pretrained(directory, device="cpu", dtype=torch.float32)
    sliced = from_pretrained(directory, device="cpu", dtype=torch.float32, tensor_parallel=tp)
    want = dict(whole.named_parameters())
    n_sliced = 0
    for name, p in sliced.named_parameters():
        kind = getattr(p, "tp_kind", None)
        got = p.detach() if kind is None else gather_full_weight(kind, p.detach(), whole.cfg, tp)
        n_sliced += kind is not None
        assert torch.equal(got, want[name].detach()), name
    assert n_sliced == 5 * whole.cfg.num_hidden_layers      # qkv, its bias, o, gate_up, down


def test_checkpoint_loads_into_tensor_parallel_slices(tmp_path):
    from halo_b200.checkpoint.save import save_model
    from halo_b200.models.qwen3 import build_model

    cfg = ModelConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=16, intermediate_size=96, moe_intermediate_size=0, num_experts=0, model_type="qwen2",
                      use_qk_norm=False, attention_bias=True)
    model = build_model(cfg, device="cpu", seed=9)
    with torch.no_grad():
        for layer in model.layers:
            layer.self_attn.qkv_bias.normal_(0.0, 0.3, generator=torch.Generator().manual_seed(2))
    d = str(tmp_path / "ckpt")
    save_model(model, d, save_dtype=None)
    run_gloo_ranks(_sliced_load_worker, 2, args=(d,), timeout=120.0)


def _leader_worker(rank, world):
    import types

    import numpy as np
    import torch.distributed as dist

    from halo_b200.runtime.collectives import share_from_leader
    from halo_b200.trainers.grpo.trainer import GRPOTrainer, Rollout

    # two tensor-parallel pairs: (0, 1) and (2, 3); every rank would sample something else
    pairs = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    mine = pairs[rank // 2]
    calls = []

    def source(i):
        calls.append(i)
        if i == 2:
            return None
        return [Rollout(np.arange(3 + rank), np.arange(2 + i), None, float(rank))]

    got = share_from_leader(lambda: source(0), mine)
    assert got[0].reward == float(2 * (rank // 2)) and len(got[0].prompt_ids) == 3 + 2 * (rank // 2)     # the pair's first rank's
    assert calls == ([0] if rank % 2 == 0 else [])                                                      # only leaders sampled
    # through the trainer's seam: a model that carries a tensor-parallel descriptor
    fake = types.SimpleNamespace(model=types.SimpleNamespace(tensor_parallel=types.SimpleNamespace(group=mine), expert_tensor_parallel=None),
                                 rollout_source=source)
    fake._sibling_group = lambda: GRPOTrainer._sibling_group(fake)
    r1 = GRPOTrainer._shared_round(fake, 1)
    assert r1[0].reward == float(2 * (rank // 2)) and len(r1[0].completion_ids) == 3
    assert GRPOTrainer._shared_round(fake, 2) is None                                                   # end of data reaches the follower too
    plain = types.SimpleNamespace(model=types.SimpleNamespace(tensor_parallel=None, expert_tensor_parallel=None), rollout_source=source)
    plain._sibling_group = lambda: GRPOTrainer._sibling_group(plain)
    assert GRPOTrainer._shared_round(plain, 0)[0].reward == float(rank)                                  # no slicing: every rank its own


def test_rollouts_come_from_the_leader_of_a_sliced_replica():
    run_gloo_ranks(_leader_worker, 4, timeout=240)
