"""Chunk planning / packing of the weight sync and the gloo broadcast path (CPU)."""

import torch

from halo_b200.weight_sync.chunking import manifest_of, pack_chunk, plan_chunks, unpack_chunk
from tests.common.gloo import run_gloo_ranks


def test_chunk_plan_round_trip():
    tensors = {"a": torch.randn(100, 7).bfloat16(), "b": torch.randn(33), "c": torch.arange(1000, dtype=torch.int32)}
    slots, sizes = plan_chunks(manifest_of(tensors.items()), chunk_bytes=2048)
    assert len(sizes) >= 2 and all(s.offset % 256 == 0 for s in slots)
    out = {k: torch.zeros_like(v) for k, v in tensors.items()}
    for c, size in enumerate(sizes):
        buf = torch.zeros(size, dtype=torch.uint8)
        pack_chunk(slots, c, tensors, buf)
        unpack_chunk(slots, c, buf, out)
    for k in tensors:
        assert torch.equal(out[k], tensors[k])


def _worker(rank, world):
    import torch.distributed as dist

    from halo_b200.weight_sync.group import BroadcastSync

    torch.manual_seed(0)
    src = {"w1": torch.randn(64, 64), "w2": torch.randn(1000)}
    sync = BroadcastSync(dist.group.WORLD, "cpu", manifest_of(src.items()), src_rank=0, chunk_bytes=4096)
    if rank == 0:
        sync.push(src)
    else:
        dst = {k: torch.zeros_like(v) for k, v in src.items()}
        sync.push(None, into=dst)
        for k in src:
            assert torch.equal(dst[k], src[k])


def test_broadcast_sync_over_gloo():
    run_gloo_ranks(_worker, 2)
