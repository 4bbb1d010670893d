"""Context parallelism on packed rows over two and four gloo ranks: layouts, and loss + gradients of the chunked
model against the same model run on the whole row by one rank."""

import numpy as np
import pytest
import torch

from halo_b200.parallel.context_parallel import make_layout
from tests.common.gloo import run_gloo_ranks


def test_balanced_layout_snaps_cuts_to_document_tiles_and_pairs_early_with_late_pieces():
    cu = np.array([0, 10, 700, 750, 2000, 2560])
    lays = [make_layout(cu, r, 2) for r in range(2)]            # four pieces; nominal cuts at 640, 1280, 1920
    assert lays[0].bounds.tolist() == [0, 650, 1262, 1902, 2560]             # 10 + 5 * 128, 750 + 4 * 128, 750 + 9 * 128
    assert lays[0].owner.tolist() == [0, 1, 1, 0] and lays[0].loc.tolist() == [0, 0, 612, 650]
    assert lays[0].rows_of_rank == [650 + 658, 612 + 640]
    assert lays[1].local_index().tolist() == list(range(650, 1902))
    assert lays[0].to_local(1902) == (0, 650) and lays[0].to_local(700) == (1, 50)
    # what a rank produces for foreign keys is exactly what the owners expect back
    for r, lay in enumerate(lays):
        for rank, my_row, n, src_row in lay.returns:
            glo = next(lo for lo, hi, srow in lays[rank].written[rank] if srow == src_row)
            assert lays[r].to_local(glo) == (r, my_row)
    assert sum(len(l.returns) for l in lays) == sum(len(w) for w in lays[0].written)
    # rank 0's late piece sees document [750, 2000) from its start: it produces dK/dV for rank 1's rows 750..1902
    assert (750, 1262, 100) in lays[0].written[0] and (1262, 1902, 612) in lays[0].written[0]
    with pytest.raises(ValueError, match="without tokens"):
        make_layout(np.array([0, 10]), 0, 4)
    contiguous = make_layout(cu, 1, 2, balance=False)
    assert contiguous.bounds.tolist() == [0, 1262, 2560] and contiguous.owner.tolist() == [0, 1]


def test_work_lists_cover_the_causal_document_mask_exactly_once():
    from halo_b200.parallel.context_parallel import build_cp_plan, covered_pairs

    rng = np.random.default_rng(0)
    for _ in range(6):
        lens = np.concatenate([rng.integers(1, 700, size=int(rng.integers(1, 6))), [1100]])
        rng.shuffle(lens)
        cu = np.concatenate([[0], np.cumsum(lens)])
        T = int(cu[-1])
        want = np.zeros((T, T), bool)
        for s, e in zip(cu[:-1], cu[1:]):
            want[s:e, s:e] = np.tril(np.ones((e - s, e - s), bool))
        for cp, balance in ((2, True), (4, True), (4, False)):
            got_q, got_k = np.zeros((T, T), bool), np.zeros((T, T), bool)
            for r in range(cp):
                lay = make_layout(cu, r, cp, balance)
                plan = build_cp_plan(lay, None)
                f, k = covered_pairs(lay, plan)
                assert not (got_q & f).any() and not (got_k & k).any()
                got_q |= f
                got_k |= k
                for item in plan.cp_items[1]:                 # a key tile and each query segment lie in one piece
                    k0, e = item[0], item[3]
                    assert lay.piece_of(k0) == lay.piece_of(min(k0 + 127, e - 1))
                    for qb, n in ((item[1], item[2]), (item[4], item[5])):
                        if n:
                            assert lay.owner[lay.piece_of(qb)] == r and (qb - k0) % 64 == 0
                            assert lay.piece_of(min(qb + 64 * n, e) - 1) == lay.piece_of(qb)
            assert (got_q == want).all() and (got_k == want).all()


def _worker(rank, world):
    import dataclasses

    import torch.distributed as dist

    from halo_b200.data.packing import pack_documents
    from halo_b200.models.config import PRESETS
    from halo_b200.models.qwen3 import build_model
    from halo_b200.parallel.context_parallel import ContextParallel, slice_batch

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), num_hidden_layers=2)
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, cfg.vocab_size, size=n) for n in (370, 900, 50, 1240)]     # 2560 tokens; documents straddle cuts
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


def test_long_document_work_is_balanced_across_ranks():
    """One long document: with paired early / late pieces every rank visits the same number of (query tile, key tile)
    pairs; contiguous chunks give the last rank several times the first rank's share."""
    from halo_b200.parallel.context_parallel import build_cp_plan

    cu = np.array([0, 16384])

    def pairs(balance):
        out = []
        for r in range(4):
            plan = build_cp_plan(make_layout(cu, r, 4, balance), None)
            out.append(sum(n64 for _, _, n64, _ in plan.cp_items[0]))
        return out

    balanced, contiguous = pairs(True), pairs(False)
    assert max(balanced) - min(balanced) <= 2 * 4          # at most the diagonal tiles differ
    assert max(contiguous) > 5 * min(contiguous)
    assert sum(balanced) == sum(contiguous)


def test_expert_parallel_times_context_parallel_through_the_entry_point(tmp_path):
    """``expert_parallel_size: 4`` with ``context_parallel_size: 2`` on four CPU ranks through the launcher (the layout of
    the 8-GPU EP8 x CP2 long-row runs, halved): two pairs of ranks each cut one row, all four shard the experts; the loss
    curve is the one of two data-parallel ranks that each hold a whole row."""
    import os
    import re
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(name, extra, n):
        cfg = tmp_path / f"{name}.yaml"
        cfg.write_text("model_preset: tiny-moe\ninit_from_scratch: true\ndataset_format: synthetic\npacked_row_length: 1024\n"
                       "doc_length_min: 200\ndoc_length_max: 700\n"
                       "max_steps: 5\nlearning_rate: 3.0e-3\nlr_scheduler_type: constant\noptim: adamw_torch\nweight_decay: 0.0\n"
                       f"max_grad_norm: 0.0\noutput_dir: {tmp_path}/{name}\nlogging_steps: 1\n" + extra)
        r = subprocess.run([sys.executable, "-m", "halo_b200.cli", "launch", "sft", str(cfg), "-n", str(n), "--port", "29741"],
                           cwd=root, capture_output=True, text=True, timeout=600,
                           env=dict(os.environ, CUDA_VISIBLE_DEVICES="", NVLINK_DOMAIN_SIZE="4"))
        out = r.stdout + r.stderr
        assert r.returncode == 0, out[-4000:]
        return [float(x) for x in re.findall(r"step \d+ loss ([0-9.]+)", out)], out

    both, out = run("ep4cp2", "expert_parallel_size: 4\ncontext_parallel_size: 2\n", 4)
    assert len(both) >= 5, out[-3000:]
    flat, _ = run("ep2", "expert_parallel_size: 2\n", 2)
    assert abs(both[0] - flat[0]) < 4e-4, (both[:2], flat[:2])
    assert max(abs(a - b) / b for a, b in zip(both[:5], flat[:5])) < 5e-3, (both, flat)
