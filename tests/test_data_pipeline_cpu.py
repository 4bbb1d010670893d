"""The coordinated data pipeline: deterministic keys (same inputs same key, a changed stage invalidates what follows),
cached rows equal freshly computed ones, a second run builds nothing, and on gloo ranks one rank per filesystem scope
does the work while the others wait and read."""

import json
import os
import types

import numpy as np
import torch

from halo_b200.data.datasets import build_sft_batches
from halo_b200.data.pipeline import Pipeline, Ragged, function_fingerprint
from tests.common.gloo import run_gloo_ranks


class CharTokenizer:
    name_or_path = "char-tokenizer"
    vocab_size = 256

    def __call__(self, text, add_special_tokens=False, **kw):
        return {"input_ids": [ord(c) % 256 for c in text]}


def _write_dataset(path, n=40):
    rng = np.random.default_rng(0)
    with open(path, "w") as f:
        for i in range(n):
            text = "".join(chr(97 + int(c)) for c in rng.integers(0, 26, size=int(rng.integers(5, 60))))
            f.write(json.dumps({"prompt": f"q{i}: ", "completion": text}) + "\n")


def _tokenize(rec):
    ids = [ord(c) % 256 for c in rec["prompt"] + rec["completion"]]
    return np.asarray(ids), np.asarray([False] * len(rec["prompt"]) + [True] * len(rec["completion"]))


def test_keys_cache_and_equality_with_the_uncached_path(tmp_path):
    data = tmp_path / "train.jsonl"
    _write_dataset(data)
    cache = str(tmp_path / "cache")

    def build(row_len=64, min_len=0):
        p = Pipeline(str(data), cache).map(_tokenize, "tokenize", tokenizer="char")
        if min_len:
            p.filter(lambda t, m: len(t) >= min_len, "min_length", min_len=min_len)
        return p.pack(row_len, "best_fit", completion_only=True, shuffle_seed=3)

    first = build()
    rows = first.rows()
    assert first.built == ["tokenize", "pack"] and len(rows) > 5
    again = build()
    rows2 = again.rows()
    assert again.built == [] and again.keys() == first.keys()                     # found, not rebuilt
    assert all(torch.equal(a.input_ids, b.input_ids) and torch.equal(a.labels, b.labels) for a, b in zip(rows, rows2))
    # another row length re-packs from the cached tokens; a filter in between re-runs from the filter on
    wider = build(row_len=128)
    wider.rows()
    assert wider.built == ["pack"] and wider.keys()[0] == first.keys()[0] and wider.keys()[1] != first.keys()[1]
    filtered = build(min_len=30)
    kept = filtered.rows()
    assert filtered.built == ["min_length", "pack"]
    report = json.load(open(os.path.join(cache, filtered.keys()[1], "stage.json")))
    assert report["dropped"] > 0 and report["documents"] + report["dropped"] == 40
    assert sum(int((r.labels != -100).sum()) for r in kept) < sum(int((r.labels != -100).sum()) for r in rows)
    # a changed function body is a changed key; touching the file is a changed source
    assert function_fingerprint(_tokenize) != function_fingerprint(lambda rec: _tokenize(rec))
    before = first.keys()[0]
    os.utime(data, (1, 1))
    assert build().keys()[0] != before
    # the ragged store round-trips types and values
    docs = [(np.arange(5), np.array([True, False, True, True, False])), (np.zeros(0, np.int64), np.zeros(0, bool))]
    Ragged.write(str(tmp_path / "r"), docs)
    back = Ragged.read(str(tmp_path / "r"))
    assert back[0][0].dtype == np.int64 and back[0][1].dtype == bool and back[0][1].tolist() == docs[0][1].tolist() and len(back[1][0]) == 0


def test_sft_batches_through_the_cache_equal_the_direct_path(tmp_path):
    data = tmp_path / "train.jsonl"
    _write_dataset(data)
    args = types.SimpleNamespace(dataset_path=str(data), dataset_format="prompt_completion", packed_row_length=96, packing_strategy="sequential",
                                 completion_only_loss=True, shuffle_seed=5, cache_dir="")
    direct = build_sft_batches(args, CharTokenizer(), dp_rank=1, dp_world=2)
    args.cache_dir = str(tmp_path / "cache")
    cached = build_sft_batches(args, CharTokenizer(), dp_rank=1, dp_world=2)
    assert len(direct) == len(cached) > 0
    for a, b in zip(direct, cached):
        assert torch.equal(a.input_ids, b.input_ids) and torch.equal(a.labels, b.labels) and torch.equal(a.position_ids, b.position_ids)
        assert a.cu_seqlens.tolist() == b.cu_seqlens.tolist() and a.n_scored == b.n_scored


def _worker(rank: int, world: int, base: str):
    os.environ.update({"LOCAL_RANK": str(rank % 2), "LOCAL_WORLD_SIZE": "2", "DIST_SHARED_FILESYSTEM": "0"})
    from halo_b200.runtime import filesystem as fs

    fs.resolve_consensus()
    # per-node storage: each "node" has its own cache directory, filled by the node's first rank only
    cache = os.path.join(base, f"cache_node{rank // 2}")
    p = Pipeline(os.path.join(base, "train.jsonl"), cache).map(_tokenize, "tokenize").pack(64)
    rows = p.rows(rank, world)
    assert p.built == (["tokenize", "pack"] if rank % 2 == 0 else []), (rank, p.built)
    assert len(rows) > 0
    fs.forget_consensus()


def test_one_rank_per_scope_builds(tmp_path):
    _write_dataset(tmp_path / "train.jsonl")
    run_gloo_ranks(_worker, 4, args=(str(tmp_path),), timeout=240)
