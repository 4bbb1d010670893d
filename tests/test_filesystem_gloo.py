"""Filesystem scope on four gloo ranks standing for two nodes of two ranks: the job-wide agreement on the sharing flags,
the writer / load rank of each scope, the store-based main-first wait, the sentinel probe in both directions and the
start-up check of the environment catalogue."""

import os
import time

import pytest

from tests.common.gloo import run_gloo_ranks


def _as_two_nodes(rank: int):
    os.environ.update({"LOCAL_RANK": str(rank % 2), "LOCAL_WORLD_SIZE": "2", "DIST_FS_PROBE_TIMEOUT_SECONDS": "1"})


def _worker(rank: int, world: int, base: str):
    from halo_b200.runtime import filesystem as fs
    from halo_b200.runtime import ranks
    from halo_b200.runtime.consensus import RankFailure, reject_divergent_environment

    _as_two_nodes(rank)
    assert ranks.get_num_nodes() == 2 and ranks.get_node_rank() == rank // 2

    # --- the flags: a multi-node job defaults to per-node; rank 3 was launched with another value and is overruled
    for k in ("DIST_SHARED_FILESYSTEM", "DIST_INPUT_SHARED_FILESYSTEM", "DIST_OUTPUT_SHARED_FILESYSTEM"):
        os.environ.pop(k, None)
    assert not fs.output_is_shared()
    os.environ["DIST_SHARED_FILESYSTEM"] = "1"
    os.environ["DIST_INPUT_SHARED_FILESYSTEM"] = "0"
    if rank == 3:
        os.environ["DIST_OUTPUT_SHARED_FILESYSTEM"] = "0"
    agreed = fs.resolve_consensus()
    assert agreed == {"DIST_SHARED_FILESYSTEM": True, "DIST_INPUT_SHARED_FILESYSTEM": False, "DIST_OUTPUT_SHARED_FILESYSTEM": True}
    assert fs.output_is_shared() and not fs.input_is_shared()                    # rank 3 too
    assert fs.is_writer_rank() == (rank == 0)                                     # shared output: one writer
    assert fs.is_load_rank() == (rank % 2 == 0)                                   # per-node input: one per node

    # --- main-first over the store, per node: the node's first rank fills its cache, its neighbour finds it filled
    cache = os.path.join(base, f"node{rank // 2}", "cache.txt")
    os.makedirs(os.path.dirname(cache), exist_ok=True)
    with fs.main_first_by_store("fill-cache") as first:
        assert first == (rank % 2 == 0)
        if first:
            time.sleep(0.3)
            with open(cache, "w") as f:
                f.write(f"built by rank {rank}")
        else:
            assert open(cache).read() == f"built by rank {rank - 1}"
    # a failure of the first rank reaches its waiters by name instead of leaving them waiting
    with pytest.raises((ValueError, RankFailure), match="no such dataset"):
        with fs.main_first_by_store("failing-fill"):
            if rank % 2 == 0:
                raise ValueError("no such dataset")

    # --- the writer creates the output directory, everyone leaves together
    out = os.path.join(base, "out", "run1")
    fs.makedirs_on_writer(out)
    assert os.path.isdir(out)

    # --- the probe: one directory all ranks see is shared; per-node directories are not
    assert fs.sentinel_visibility(out) == [True] * world
    fs.verify_filesystem_sharing(out, True, "output")
    with pytest.raises(RankFailure, match="declared per-node, but all 4 ranks see"):
        fs.verify_filesystem_sharing(out, False, "output")
    mine = os.path.join(base, f"disk_of_node{rank // 2}")
    os.makedirs(mine, exist_ok=True)
    assert fs.sentinel_visibility(mine) == [True, True, False, False]
    fs.verify_filesystem_sharing(mine, False, "input")
    with pytest.raises(RankFailure, match="declared shared, but 2 of 4 ranks .first: rank 2."):
        fs.verify_filesystem_sharing(mine, True, "input")
    fs.verify_job_directories(out, {"datasets": mine})

    # --- the environment catalogue must read the same everywhere, except for the per-rank knobs
    os.environ["HALO_LOG_LEVEL"] = "DEBUG" if rank == 1 else "INFO"             # per rank: allowed
    os.environ.pop("DIST_OUTPUT_SHARED_FILESYSTEM", None)
    reject_divergent_environment()
    if rank == 2:
        os.environ["HALO_MOE_FUSED"] = "0"
    with pytest.raises(RankFailure, match="HALO_MOE_FUSED: '0' on ranks .2., unset on ranks .0, 1, 3."):
        reject_divergent_environment()
    fs.forget_consensus()


def test_filesystem_scope_on_two_emulated_nodes(tmp_path):
    run_gloo_ranks(_worker, 4, args=(str(tmp_path),), timeout=240)


def test_contradiction_messages():
    from halo_b200.runtime.filesystem import contradiction

    assert contradiction("output", "/x", True, [True, True]) is None
    assert contradiction("output", "/x", False, [True, False]) is None
    assert "could not read back" in contradiction("output", "/x", True, [False, True])
    assert "DIST_OUTPUT_SHARED_FILESYSTEM=0" in contradiction("output", "/x", True, [True, False])
    assert "DIST_INPUT_SHARED_FILESYSTEM=1" in contradiction("input", "/x", False, [True, True])
    assert contradiction("input", "/x", True, []) is None
