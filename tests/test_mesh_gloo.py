"""DeviceMesh builders and DTensor views on four gloo ranks: axis groups of the 1-D, hybrid-sharding and (dp, tp) meshes
hold the ranks the layout promises, whole-job checks refuse partial meshes, and a hand-held shard round-trips through
its DTensor view."""

import pytest
import torch

from tests.common.gloo import run_gloo_ranks


def _worker(rank: int, world: int):
    import torch.distributed as dist

    from halo_b200.parallel import mesh as M

    dp = M.build_dp_mesh(world, device_type="cpu")
    assert M.mesh_dim_names(dp) == ("dp",) and dist.get_world_size(M.dp_group(dp)) == world
    assert M.shard_and_replicate_groups(dp)[1] is None and M.tp_group(dp) is None
    hs = M.build_dp_mesh(world, dp_replicate_size=2, device_type="cpu")
    shard, rep = M.shard_and_replicate_groups(hs)
    # row-major (dp_replicate, dp_shard): consecutive ranks share a shard group, ranks two apart share a slice
    assert dist.get_process_group_ranks(shard) == ([0, 1] if rank < 2 else [2, 3])
    assert dist.get_process_group_ranks(rep) == ([0, 2] if rank % 2 == 0 else [1, 3])
    with pytest.raises(ValueError):
        M.build_dp_mesh(world, dp_replicate_size=3, device_type="cpu")
    with pytest.raises(ValueError):
        M.build_dp_mesh(world // 2, device_type="cpu")                      # a partial mesh without its own group
    tp = M.build_dp_tp_mesh(2, dp_size=world // 2, device_type="cpu")
    assert dist.get_process_group_ranks(M.tp_group(tp)) == ([0, 1] if rank < 2 else [2, 3])
    assert dist.get_process_group_ranks(M.dp_group(tp)) == ([0, 2] if rank % 2 == 0 else [1, 3])
    # a slice held by hand, seen as a DTensor: sharded over dp_shard, replicated over dp_replicate
    full = torch.arange(8 * 3, dtype=torch.float32).view(8, 3)
    mine = full[4 * (rank % 2):4 * (rank % 2) + 4].clone()
    dt = M.as_dtensor(mine, hs, 0, M.MeshDim.DP_SHARD)
    assert tuple(dt.shape) == (8, 3) and torch.equal(M.to_local(dt), mine)
    assert torch.equal(M.full_tensor(dt), full)
    assert torch.equal(M.full_tensor(mine), mine) and M.to_local(mine) is mine
    bank = torch.full((2, 5), float(rank))
    ep = M.expert_bank_dtensor(bank, dist.group.WORLD, "cpu")
    assert tuple(ep.shape) == (2 * world, 5) and M.full_tensor(ep)[2 * rank, 0] == rank


def test_meshes_and_dtensor_views_on_four_ranks():
    run_gloo_ranks(_worker, 4, timeout=240)
