"""Attention work lists on the host: every (query, key) pair the mask allows is visited exactly once by the query-tile list
and by the key-tile list, without and with a sliding window."""

import numpy as np
import pytest

from halo_b200.ops.attention import build_plan


def _lists(cu, window):
    """The lists build_plan uploads (kept on the host as well)."""

    plan = build_plan(cu, None, window=window)
    assert plan.fwd is None and plan.window == window
    return plan.host_lists["bwd_q"], plan.host_lists["bwd_kv"]


@pytest.mark.parametrize("window", [0, 64, 100, 128, 300, 4096])
def test_lists_cover_the_mask_exactly_once(window):
    rng = np.random.default_rng(window)
    lens = rng.integers(1, 900, size=5)
    cu = np.concatenate([[0], np.cumsum(lens)])
    T = int(cu[-1])
    want = np.zeros((T, T), bool)
    for s, e in zip(cu[:-1], cu[1:]):
        n = e - s
        m = np.tril(np.ones((n, n), bool))
        if window:
            m &= ~np.tril(np.ones((n, n), bool), -window)
        want[s:e, s:e] = m
    bq, bkv = _lists(cu, window)
    got_q = np.zeros((T, T), bool)
    for q0, k_first, n64, e in bq:
        for q in range(q0, min(q0 + 128, e)):
            for k in range(k_first, min(k_first + 64 * n64, e)):
                if k <= q and (not window or q - k < window):
                    assert not got_q[q, k]
                    got_q[q, k] = True
    got_k = np.zeros((T, T), bool)
    for k0, qb, nq, e in bkv:
        for k in range(k0, min(k0 + 128, e)):
            for q in range(qb, min(qb + 64 * nq, e)):
                if k <= q and (not window or q - k < window):
                    assert not got_k[q, k]
                    got_k[q, k] = True
    assert (got_q == want).all() and (got_k == want).all()
    if window:
        # the lists are cut to the window: no query tile walks more key tiles than a window plus its own rows need
        assert max(n64 for _, _, n64, _ in bq) <= (window + 127 + 63) // 64 + 1


def test_reference_applies_the_window():
    import torch

    from halo_b200.ops.attention import attention_reference

    torch.manual_seed(0)
    q, k, v = torch.randn(40, 2 * 16), torch.randn(40, 16), torch.randn(40, 16)
    full = attention_reference(q, k, v, [0, 40], 2, 1)
    wide = attention_reference(q, k, v, [0, 40], 2, 1, window=64)
    narrow = attention_reference(q, k, v, [0, 40], 2, 1, window=4)
    assert torch.allclose(full, wide) and not torch.allclose(full, narrow)
    assert torch.allclose(full[:4], narrow[:4])          # the first `window` rows see everything before them anyway


def test_windowed_models_are_sent_to_the_flash_kernels_only_where_they_run():
    import dataclasses

    import torch

    from halo_b200.models.attention_selection import attention_path
    from halo_b200.models.config import PRESETS

    cfg = dataclasses.replace(PRESETS["tiny-moe"](), sliding_window=64, head_dim=128)
    assert attention_path(cfg, "cuda", torch.bfloat16)[0] == "flash"
    assert "sliding_window=64" in attention_path(cfg, "cuda", torch.bfloat16)[1]
    assert attention_path(cfg, "cpu", torch.float32)[0] == "masked"
    assert attention_path(cfg, "cuda", torch.float32)[0] == "masked"
    assert attention_path(dataclasses.replace(cfg, head_dim=64), "cuda", torch.bfloat16)[0] == "masked"
    assert attention_path(dataclasses.replace(cfg, attention_sinks=True), "cuda", torch.bfloat16)[0] == "masked"
    assert attention_path(cfg, "cuda", torch.bfloat16, tree_packing=True)[0] == "masked"
