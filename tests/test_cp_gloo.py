"""Context parallelism on packed rows over two and four gloo ranks: layouts, and loss + gradients of the chunked
model against the same model run on the whole row by one rank."""

import numpy as np
import pytest
import torch

from halo_b200.parallel.context_parallel import make_layout
from tests.common.gloo import run_gloo_ranks


def test_layout_sources_and_returns_are_mirror_images():
    cu = np.array([0, 10, 70, 75, 200, 256])
    lays = [make_layout(cu, r, 4) for r in range(4)]          # chunks of 64 tokens
    assert [(l.lo, l.hi, l.p0) for l in lays] == [(0, 64, 0), (64, 128, 10), (128, 192, 75), (192, 256, 75)]
    assert lays[1].sources == [(0, 10, 54, 0)] and lays[1].cu_ext.tolist() == [0, 60, 65, 118]
    assert lays[3].sources == [(1, 11, 53, 0), (2, 0, 64, 53)]
    for r, l in enumerate(lays):                               # every pull has its matching gradient return
        for s, src_row, n, dst_row in l.sources:
            assert (r, src_row, n, dst_row) in lays[s].returns
    assert sum(len(l.returns) for l in lays) == sum(len(l.sources) for l in lays)
    with pytest.raises(ValueError):
        make_layout(np.array([0, 10]), 0, 4)


def _worker(rank, world):
    import dataclasses

    import torch.distributed as dist

    from halo_b200.data.packing import pack_documents
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.context_parallel import ContextParallel, slice_batch

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2)
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, cfg.vocab_size, size=n) for n in (37, 90, 5, 124)]     # 256 tokens; documents straddle cuts
    full_batch = pack_documents(docs)
    norm = float(full_batch.n_scored)

    model = build_model(cfg, device="cpu", dtype=torch.float32, seed=3)
    model.context_parallel = ContextParallel(dist.group.WORLD, "cpu", cfg, full_batch.n_tokens)
    b = slice_batch(full_batch, rank, world)
    loss = model(b.input_ids, b.position_ids, b.cu_seqlens, b.labels, norm)
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)
    grads = {}
    for n, p in model.named_parameters():
        g = p.grad.clone()
        dist.all_reduce(g)                 # chunks of a row are like data-parallel shards for the weights
        grads[n] = g

    ref = build_model(cfg, device="cpu", dtype=torch.float32, seed=3)
    ref_loss = ref(full_batch.input_ids, full_batch.position_ids, full_batch.cu_seqlens, full_batch.labels, norm)
    ref_loss.backward()
    assert torch.allclose(total, ref_loss.detach(), rtol=1e-5, atol=1e-6), (float(total), float(ref_loss))
    for n, p in ref.named_parameters():
        assert torch.allclose(grads[n], p.grad, rtol=2e-4, atol=2e-6), n


@pytest.mark.parametrize("world", [2, 4])
def test_chunked_row_matches_whole_row(world):
    run_gloo_ranks(_worker, world, timeout=120.0)
