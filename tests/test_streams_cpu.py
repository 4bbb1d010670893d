"""Residual-stream ops on CPU: every op's closed-form backward against autograd of the plain expression, the
Sinkhorn projection's invariants, and the masked-softmax backward against autograd of a masked softmax."""

import pytest
import torch

from halo_b200.ops import streams as S

torch.manual_seed(0)


def grads(fn, *inputs):
    xs = [x.detach().clone().requires_grad_(True) for x in inputs]
    out = fn(*xs)
    weight = torch.randn(out.shape, generator=torch.Generator().manual_seed(5))
    (out.float() * weight).sum().backward()
    return out.detach(), [x.grad for x in xs]


def check(op, ref, *inputs, tol=1e-5):
    out_a, g_a = grads(op, *inputs)
    out_b, g_b = grads(ref, *inputs)
    assert torch.allclose(out_a.float(), out_b.float(), atol=tol, rtol=tol)
    for i, (a, b) in enumerate(zip(g_a, g_b)):
        assert a is not None and torch.allclose(a, b, atol=tol * 10, rtol=tol * 10), (i, (a - b).abs().max())


@pytest.mark.parametrize("N", [1, 2, 4, 8])
def test_collapse_mix_inject(N):
    T, H = 6, 16
    stream, block = torch.randn(2, T, N, H), torch.randn(2, T, H)
    w, post, gate = torch.rand(2, T, N), torch.rand(2, T, N), torch.randn(2, T, N)
    comb = torch.rand(2, T, N, N)
    check(S.collapse_streams, S.collapse_streams_reference, stream, w)
    check(S.mix_streams, S.mix_streams_reference, block, stream, post, comb)
    check(S.inject_streams, S.inject_streams_reference, block, stream, gate)


@pytest.mark.parametrize("N,iters", [(2, 1), (4, 3), (4, 20), (8, 5)])
def test_sinkhorn(N, iters):
    comb = torch.softmax(torch.randn(3, 5, N, N), dim=-1) + 1e-6
    check(lambda c: S.sinkhorn_knopp(c, iters, 1e-6), lambda c: S.sinkhorn_knopp_reference(c, iters, 1e-6), comb, tol=1e-5)
    out = S.sinkhorn_knopp(comb, 30, 1e-6)
    assert torch.allclose(out.sum(-2), torch.ones(3, 5, N), atol=1e-4)          # columns sum to one after a column pass
    assert torch.allclose(out.sum(-1), torch.ones(3, 5, N), atol=1e-2)          # rows nearly so
    assert not S.sinkhorn_knopp(comb, 2, 1e-6).requires_grad


def test_projection():
    T, N, H, K = 7, 4, 16, 4 * 4 + 2 * 4
    stream, fn = torch.randn(T, N, H), torch.randn(K, N * H) * 0.1
    check(lambda s, f: S.project_streams(s, f, 1e-6), lambda s, f: S.project_streams_reference(s, f, 1e-6), stream, fn, tol=1e-5)


@pytest.mark.parametrize("streams", [1, 2, 4])
def test_grouped_rms_norm_and_gate_mix(streams):
    rows, H, rank = 9, 16, 8
    x, w = torch.randn(rows, streams * H), torch.randn(streams * H) * 0.1
    check(lambda a, b: S.grouped_rms_norm(a, b, 1e-6, streams), lambda a, b: S.grouped_rms_norm_reference(a, b, 1e-6, streams), x, w)
    normed, down, w_up = torch.randn(rows, streams * H), torch.randn(rows, rank), torch.randn(streams * H, rank) * 0.3
    check(lambda a, b, c: S.gate_mix(a, b, c, streams), lambda a, b, c: S.gate_mix_reference(a, b, c, streams), normed, down, w_up)


def test_masked_softmax_backward_matches_autograd():
    heads, Q, K, scale = 3, 5, 11, 0.37
    scores = torch.randn(heads, Q, K, requires_grad=True)
    allowed = torch.rand(Q, K) > 0.3
    allowed[:, 0] = True
    masked = (scores * scale).masked_fill(~allowed, float("-inf"))
    probs = torch.softmax(masked, dim=-1)
    upstream = torch.randn(heads, Q, K)
    (probs * upstream).sum().backward()
    lse = torch.logsumexp(masked, dim=-1).detach()
    delta = (probs * upstream).sum(-1).detach()
    p, d = S.masked_softmax_backward(scores.detach(), allowed, lse, scale, upstream, delta, True, torch.float32)
    assert torch.allclose(p, probs.detach(), atol=1e-6)
    assert torch.allclose(d, scores.grad, atol=1e-6)
    p_only, none = S.masked_softmax_backward(scores.detach(), allowed, lse, scale, writes_probs=True, dtype=torch.float32)
    assert none is None and torch.equal(p_only, p)


def test_shape_guards():
    with pytest.raises(ValueError, match="weight of shape"):
        S.collapse_streams(torch.randn(3, 4, 8), torch.randn(3, 3))
    with pytest.raises(ValueError, match="built for 1..8"):
        S.collapse_streams(torch.randn(3, 9, 8), torch.randn(3, 9))


def test_block_sparse_attention_matches_the_dense_mask():
    from halo_b200.ops.block_sparse_attention import block_sparse_attention, dense_reference, key_positions

    g = torch.Generator().manual_seed(0)
    ratio, topk, Hq, Hkv, D = 4, 3, 4, 2, 16
    docs = [23, 9, 2]
    T = sum(docs)
    first = torch.cat([torch.full((n,), s) for n, s in zip(docs, [0, 23, 32])])
    visible = torch.cat([torch.arange(1, n + 1) for n in docs])
    spans = torch.stack([first, visible], dim=1)
    blocks = torch.zeros(T, topk, dtype=torch.int64)
    for t in range(T):
        complete = int(visible[t]) // ratio
        if complete:
            pick = torch.randperm(complete, generator=g)[:topk]
            blocks[t, :len(pick)] = pick                     # distinct blocks; unused slots keep 0 and are masked by the count
    pos, ok = key_positions(spans, blocks, ratio)
    assert (pos[ok] < (first + visible)[:, None].expand_as(pos)[ok]).all()          # never a key from the future or another document
    assert int(ok[0].sum()) == 1 and int(ok[22].sum()) == min(5, topk) * ratio + 3
    q, k, v = (torch.randn(T, h, D, generator=g, requires_grad=True) for h in (Hq, Hkv, Hkv))
    got = block_sparse_attention(q, k, v, spans, blocks, ratio, chunk_queries=7)
    want = dense_reference(q, k, v, spans, blocks, ratio)
    assert torch.allclose(got, want, atol=1e-5)
    w = torch.randn(got.shape, generator=g)
    ga = torch.autograd.grad((got * w).sum(), (q, k, v))
    gb = torch.autograd.grad((want * w).sum(), (q, k, v))
    for a, b in zip(ga, gb):
        assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("kind", ["random", "tree", "window"])
def test_masked_attention_closed_form_backward(kind):
    from halo_b200.ops.masked_attention import masked_attention, masked_attention_reference, tree_mask, window_mask

    g = torch.Generator().manual_seed(3)
    Q, Hq, Hkv, D = 37, 4, 2, 16
    if kind == "random":
        allowed = torch.rand(Q, Q, generator=g) > 0.5
        allowed[5] = False                                                  # a query that sees nothing
    elif kind == "tree":
        # a 10-token prompt with three completions branching off its end
        parent = torch.tensor(list(range(-1, 9)) + [9] + list(range(10, 18)) + [9] + list(range(19, 27)) + [9] + list(range(28, 36)))
        allowed = tree_mask(parent)
        assert allowed[36, :10].all() and not allowed[36, 10:28].any() and allowed[36, 28:].all()
    else:
        allowed = window_mask([0, 20, 37], 6)
        assert allowed[25, 20:26].all() and not allowed[25, :20].any() and int(allowed[19].sum()) == 6
    q = torch.randn(Q, Hq, D, generator=g, requires_grad=True)
    k, v = (torch.randn(Q, Hkv, D, generator=g, requires_grad=True) for _ in range(2))
    got = masked_attention(q, k, v, allowed, scores_per_tile=Hq * Q * 8)     # several query tiles
    want = masked_attention_reference(q, k, v, allowed)
    assert torch.allclose(got, want, atol=1e-5)
    w = torch.randn(got.shape, generator=g)
    for a, b in zip(torch.autograd.grad((got * w).sum(), (q, k, v)), torch.autograd.grad((want * w).sum(), (q, k, v))):
        assert torch.allclose(a, b, atol=1e-5)
    # with attention sinks: one learned logit per head joins every softmax
    sinks = torch.randn(Hq, generator=g, requires_grad=True)
    got = masked_attention(q, k, v, allowed, scores_per_tile=Hq * Q * 8, sinks=sinks)
    want = masked_attention_reference(q, k, v, allowed, sinks=sinks)
    assert torch.allclose(got, want, atol=1e-5) and not torch.allclose(got, masked_attention(q, k, v, allowed), atol=1e-3)
    for a, b in zip(torch.autograd.grad((got * w).sum(), (q, k, v, sinks)), torch.autograd.grad((want * w).sum(), (q, k, v, sinks))):
        assert torch.allclose(a, b, atol=1e-5)
    # tanh soft-capping of the scores (a cap small enough to bend them)
    got = masked_attention(q * 3, k, v, allowed, scores_per_tile=Hq * Q * 8, softcap=1.5)
    want = masked_attention_reference(q * 3, k, v, allowed, softcap=1.5)
    assert torch.allclose(got, want, atol=1e-5) and not torch.allclose(got, masked_attention(q * 3, k, v, allowed), atol=1e-3)
    for a, b in zip(torch.autograd.grad((got * w).sum(), (q, k, v)), torch.autograd.grad((want * w).sum(), (q, k, v))):
        assert torch.allclose(a, b, atol=1e-5)
