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
    assert attention_path(dataclasses.replace(cfg, head_dim=64), "cuda", torch.bfloat16)[0] == "flash"
    assert attention_path(dataclasses.replace(cfg, head_dim=256), "cuda", torch.bfloat16)[0] == "masked"
    sinks = dataclasses.replace(cfg, attention_sinks=True, head_dim=64)
    assert attention_path(sinks, "cuda", torch.bfloat16)[0] == "flash"
    assert "zero-padded" in attention_path(sinks, "cuda", torch.bfloat16)[1]
    assert attention_path(sinks, "cpu", torch.float32)[0] == "masked"
    assert attention_path(dataclasses.replace(cfg, attn_logit_softcapping=50.0), "cuda", torch.bfloat16)[0] == "masked"
    assert attention_path(cfg, "cuda", torch.bfloat16, tree_packing=True)[0] == "masked"


def test_sinks_in_the_reference_and_their_gradient_from_lse_and_delta():
    """The flash path adds the sink logit to the denominator in the forward kernel and forms the sink gradient from the
    stored log-sum-exp and the backward's delta; both statements are checked here against autograd on the oracle."""
    import torch

    from halo_b200.ops.attention import _sink_grad, attention_reference
    from halo_b200.ops.masked_attention import masked_attention_reference, window_mask

    torch.manual_seed(0)
    Hq, Hkv, D, cu, window = 4, 2, 16, [0, 37, 90], 12
    T = cu[-1]
    q = torch.randn(T, Hq * D, dtype=torch.float64).requires_grad_()
    k = torch.randn(T, Hkv * D, dtype=torch.float64).requires_grad_()
    v = torch.randn(T, Hkv * D, dtype=torch.float64).requires_grad_()
    sinks = torch.randn(Hq, dtype=torch.float64).requires_grad_()
    o = attention_reference(q, k, v, cu, Hq, Hkv, window=window, sinks=sinks)
    want = masked_attention_reference(q.float().reshape(T, Hq, D), k.float().reshape(T, Hkv, D), v.float().reshape(T, Hkv, D),
                                      window_mask(np.asarray(cu), window), sinks=sinks.float())
    assert (o.float() - want.reshape(T, Hq * D)).abs().max().item() < 1e-4
    do = torch.randn_like(o)
    o.backward(do)
    # lse over keys and sink, delta = rowsum(dO * O), per head and row, as the kernels store them
    with torch.no_grad():
        rep = Hq // Hkv
        lse = torch.empty(Hq, T, dtype=torch.float64)
        for s0, e0 in zip(cu[:-1], cu[1:]):
            n = e0 - s0
            qq = q[s0:e0].reshape(n, Hq, D).transpose(0, 1)
            kk = k[s0:e0].reshape(n, Hkv, D).transpose(0, 1).repeat_interleave(rep, dim=0)
            sc = (qq @ kk.transpose(1, 2)) * D**-0.5
            mask = torch.ones(n, n, dtype=torch.bool).tril() & ~torch.ones(n, n, dtype=torch.bool).tril(-window)
            sc = sc.masked_fill(~mask, float("-inf"))
            lse[:, s0:e0] = torch.logsumexp(torch.cat([sc, sinks[:, None, None].expand(-1, n, 1)], dim=-1), dim=-1)
        delta = (do * o).reshape(T, Hq, D).sum(-1).t()
        got = _sink_grad(sinks.detach(), lse, delta)
    assert (got - sinks.grad).abs().max().item() < 1e-5      # the oracle works in fp32


def test_zero_padded_heads_leave_attention_unchanged():
    import torch

    from halo_b200.ops.attention import HEAD_DIM, _pad_heads, attention_reference

    torch.manual_seed(1)
    Hq, Hkv, D, cu = 4, 2, 64, [0, 50, 81]
    T = cu[-1]
    q, k, v = torch.randn(T, Hq * D), torch.randn(T, Hkv * D), torch.randn(T, Hkv * D)
    want = attention_reference(q, k, v, cu, Hq, Hkv)
    wide = attention_reference(_pad_heads(q, Hq, D), _pad_heads(k, Hkv, D), _pad_heads(v, Hkv, D), cu, Hq, Hkv, scale=D**-0.5)
    got = wide.reshape(T, Hq, HEAD_DIM)[:, :, :D].reshape(T, Hq * D)
    assert (got - want).abs().max().item() < 1e-5
    assert wide.reshape(T, Hq, HEAD_DIM)[:, :, D:].abs().max().item() == 0.0
