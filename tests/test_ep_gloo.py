"""Tiny Qwen3-MoE SFT on CPU: two gloo ranks with expert parallelism 2 follow the same loss curve as
one process that sees the whole batch (the plumbing configuration: 4 layers, hidden 256, 8 experts of
width 128, top-2, vocab 4096, fp32, packed 512-token rows, micro-batch 2 per rank, AdamW 1e-4, 20 steps)."""

import numpy as np
import pytest
import torch

from halo_b200.data.packing import pack_documents
from halo_b200.models.config import tiny_moe_config
from tests.common.gloo import run_gloo_ranks

STEPS = 20
ROWS_PER_RANK = 2
ROW_LEN = 512


def _rows(step: int, n_rows: int, first_row: int):
    """Rows ``first_row .. first_row + n_rows`` of the global batch of ``step`` as one packed stream."""
    docs = []
    for r in range(first_row, first_row + n_rows):
        rng = np.random.default_rng(1000 * step + r)
        left = ROW_LEN
        while left > 0:
            n = min(left, int(rng.integers(32, 257)))
            docs.append(rng.integers(0, 4096, size=n))
            left -= n
    return pack_documents(docs)


def _train(rank: int, world: int, out_path: str):
    import torch.distributed as dist

    from halo_b200.models.qwen3 import build_model
    from halo_b200.trainers.engine import TrainEngine

    torch.manual_seed(0)
    cfg = tiny_moe_config()
    transport = parallel = None
    if world > 1:
        from halo_b200.parallel.expert_parallel import CollectiveTransport
        from halo_b200.parallel.runtime import ParallelRuntime

        transport = CollectiveTransport(dist.group.WORLD)
        parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD, ep_group=dist.group.WORLD, transport=transport)
    model = build_model(cfg, device="cpu", seed=0, transport=transport, gradient_checkpointing=True)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    eng = TrainEngine(model, opt, "cpu", max_grad_norm=1.0, parallel=parallel)
    losses = []
    for step in range(STEPS):
        batch = _rows(step, ROWS_PER_RANK * (1 if world > 1 else 2), rank * ROWS_PER_RANK)
        out = eng.train_step(batch)
        loss = out.loss.reshape(-1)[0].clone()
        if world > 1:
            dist.all_reduce(loss)  # each rank's loss is its share of the globally normalised sum
        losses.append(float(loss))
    if rank == 0:
        np.save(out_path, np.asarray(losses))


def test_ep2_matches_ep1_loss_curve(tmp_path):
    single = str(tmp_path / "single.npy")
    ep2 = str(tmp_path / "ep2.npy")
    _train(0, 1, single)
    run_gloo_ranks(_train, 2, args=(ep2,), timeout=600)
    a, b = np.load(single), np.load(ep2)
    assert a.shape == b.shape == (STEPS,)
    assert abs(a[0] - np.log(4096)) < 0.2
    assert np.max(np.abs(a - b)) < 5e-3, (a, b)


def _trace_worker(rank, world):
    """Two training steps under expert parallelism with the collectives recorded: every rank enters the same
    collectives in the same order, and the second step repeats the first (nothing depends on the data)."""
    import torch
    import torch.distributed as dist

    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.models.config import tiny_moe_config
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.expert_parallel import CollectiveTransport
    from halo_b200.parallel.runtime import ParallelRuntime
    from halo_b200.trainers.engine import TrainEngine
    from tests.common.collective_recorder import recording

    cfg = tiny_moe_config()
    transport = CollectiveTransport(dist.group.WORLD)
    parallel = ParallelRuntime("cpu", dp_group=dist.group.WORLD, ep_group=dist.group.WORLD, transport=transport)
    model = build_model(cfg, device="cpu", seed=0, transport=transport)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    engine = TrainEngine(model, opt, "cpu", parallel=parallel)
    steps = []
    for step in range(2):
        # ranks see different rows with different token counts and routing: the trace must not depend on them
        batch = synthetic_packed_batch(96 + 32 * rank, cfg.vocab_size, seed=10 * step + rank, lo=8, hi=40)
        with recording() as trace:
            engine.train_step(batch)
        steps.append([(name, n) for name, n, _ in trace])
    assert steps[0] == steps[1], "the second step entered different collectives than the first"
    everyone = [None] * world
    dist.all_gather_object(everyone, steps[0])
    assert all(t == everyone[0] for t in everyone), "ranks entered different collectives"
    names = [name for name, _ in steps[0]]
    per_layer = 4 * 2          # forward pass, recomputation and backward of a layer each exchange counts and rows
    assert len(names) >= cfg.num_hidden_layers * per_layer and "all_reduce" in names


def test_collective_order_is_rank_uniform_and_static():
    from tests.common.gloo import run_gloo_ranks

    run_gloo_ranks(_trace_worker, 2, timeout=180.0)


def _negative_control_worker(rank, world):
    """The expert-parallel layer equals the undistributed one - and the bound that says so can fail: with this rank's
    experts rotated by one place the same comparison is off by orders of magnitude."""
    import torch.distributed as dist

    from halo_b200.ops.moe import moe_experts, moe_ffn_reference, router_topk
    from halo_b200.parallel.expert_parallel import CollectiveTransport

    g = torch.Generator().manual_seed(7)                       # the same on every rank: the full banks
    T, H, F, E, k = 48 + 16 * rank, 64, 32, 8, 2
    gate_up, down = torch.randn(E, 2 * F, H, generator=g) * 0.2, torch.randn(E, H, F, generator=g) * 0.2
    mine = torch.Generator().manual_seed(100 + rank)           # this rank's own tokens
    x = torch.randn(T, H, generator=mine)
    idx, w = router_topk(torch.randn(T, E, generator=mine), k, True)
    want = moe_ffn_reference(x, idx, w, gate_up, down, 0)
    per = E // world
    local_gu, local_dn = gate_up[rank * per:(rank + 1) * per].clone(), down[rank * per:(rank + 1) * per].clone()
    transport = CollectiveTransport(dist.group.WORLD)
    got = moe_experts(x, idx, w, local_gu, local_dn, transport)
    tol = 1e-5
    assert (got - want).abs().max() < tol
    wrong = moe_experts(x, idx, w, local_gu.roll(1, 0), local_dn.roll(1, 0), transport)
    assert (wrong - want).abs().max() > 1e3 * tol


def test_expert_parallel_layer_with_a_wrong_expert_negative_control():
    run_gloo_ranks(_negative_control_worker, 2, timeout=120.0)


def _latent_family_worker(rank, world, directory):
    """DeepSeek-V3 shape under expert parallelism 2: each rank loads its experts from a hub-layout checkpoint, and the loss
    of the whole batch equals the undistributed model's."""
    import torch.distributed as dist

    from halo_b200.checkpoint.load import from_pretrained
    from halo_b200.data.packing import synthetic_packed_batch
    from halo_b200.parallel.expert_parallel import CollectiveTransport

    whole = from_pretrained(directory, device="cpu", dtype=torch.float32, gradient_checkpointing=False)
    sharded = from_pretrained(directory, device="cpu", dtype=torch.float32, gradient_checkpointing=False,
                              transport=CollectiveTransport(dist.group.WORLD))
    assert sharded.layers[1].mlp.experts_gate_up.shape[0] == whole.cfg.num_experts // world
    batch = synthetic_packed_batch(64 + 16 * rank, whole.cfg.vocab_size, seed=rank, lo=8, hi=30)
    outs = []
    for m in (whole, sharded):
        out = m(batch.input_ids, batch.position_ids, batch.cu_seqlens, batch.labels)
        loss = (out.loss if hasattr(out, "loss") else out).sum()
        loss.backward()
        outs.append(loss.detach())
    assert torch.allclose(outs[0], outs[1], atol=1e-5), outs
    a, b = whole.layers[1].self_attn.kv_b_proj.grad, sharded.layers[1].self_attn.kv_b_proj.grad
    assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("family", ["deepseek_v3", "mistral4"])       # the second stores each expert bank as ONE tensor
def test_latent_attention_family_under_expert_parallelism(tmp_path, family):
    from halo_b200.checkpoint.save import save_model
    from halo_b200.models.qwen3 import build_model
    from tests.test_families_cpu import family_config

    model = build_model(family_config(family), device="cpu", seed=9, gradient_checkpointing=False)
    save_model(model, str(tmp_path / "ckpt"), save_dtype=None)
    run_gloo_ranks(_latent_family_worker, 2, args=(str(tmp_path / "ckpt"),), timeout=240.0)
