"""Push parity: after the first weight push the trainers and a rollout rank score one fixed row of tokens with the
weights they hold; a gap between the two sets of log-probabilities past a tolerance fails the run before any
rollout sampled from a mis-synchronised copy is trained on (halo/trainers/grpo/rollout/push_parity.py:1-109).

The row is derived from a seed, so both sides build it without talking; the rollout rank publishes its
log-probabilities through the rendezvous store, the trainers compare (every trainer rank scores the row - under
expert parallelism the forward is collective - and rank 0's verdict is what raises)."""

from __future__ import annotations

import pickle
import time

import numpy as np
import torch

KEY = "halo/push_parity/logprobs"


def fixed_row(vocab_size: int, length: int = 96, seed: int = 20240229):
    from halo_b200.data.packing import pack_documents

    rng = np.random.default_rng(seed)
    cut = length // 3
    return pack_documents([rng.integers(0, vocab_size, size=cut), rng.integers(0, vocab_size, size=length - cut)])


@torch.no_grad()
def score_fixed_row(model, device) -> np.ndarray:
    b = fixed_row(model.cfg.vocab_size).to(device)
    was_training = model.training
    logp, _ = model.token_logprobs(b.input_ids, b.position_ids, b.cu_seqlens, b.labels)
    model.train(was_training)
    scored = (b.labels.reshape(-1) != -100)
    return logp[scored].float().cpu().numpy()


def publish(store, logps: np.ndarray) -> None:
    store.set(KEY, pickle.dumps(logps))


def compare(store, mine: np.ndarray, tolerance: float = 0.05, timeout_seconds: float = 600.0) -> float:
    """Returns the largest absolute gap; raises when it passes ``tolerance`` or the rollout side never answers."""
    deadline = time.monotonic() + timeout_seconds
    while True:
        try:
            if store.check([KEY]):
                break
        except RuntimeError:
            pass
        if time.monotonic() > deadline:
            raise TimeoutError(f"no rollout rank published its parity scores within {timeout_seconds:.0f} s")
        time.sleep(0.02)
    theirs = pickle.loads(store.get(KEY))
    if theirs.shape != mine.shape:
        raise RuntimeError(f"push parity: the rollout side scored {theirs.shape[0]} tokens, the trainers {mine.shape[0]}")
    gap = float(np.abs(theirs - mine).max())
    if not np.isfinite(gap) or gap > tolerance:
        raise RuntimeError(f"push parity failed: after the first weight push the rollout copy's log-probabilities differ from the "
                           f"trainers' by up to {gap:.4f} nats (tolerance {tolerance}): the copies are not the same model")
    return gap
