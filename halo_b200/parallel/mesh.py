"""``DeviceMesh`` builders, mesh accessors and the DTensor view of the framework's explicitly sharded state.

The framework shards by hand (expert banks by expert, the replicated parameters' optimizer state by flat slices,
tensor-parallel weights by rows / columns), but it describes those layouts in PyTorch's own vocabulary so that code
written against FSDP2 / DTensor can read them: a 1-D ``(dp,)`` mesh, the 2-D hybrid-sharding mesh
``(dp_replicate, dp_shard)`` and the 2-D ``(dp, tp)`` mesh are built here, process groups for every axis come out of
them, and a locally held shard can be wrapped as a ``DTensor`` with the right placement (and gathered through it).

Expert- and context-parallel groups are not mesh axes: their rank orders are built by hand
(:mod:`halo_b200.parallel.layout`), as in the reference.

Counterpart of halo/distributed/mesh.py:32-114 and halo/distributed/dtensor.py.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh


class MeshDim:
    """Canonical mesh axis names. A row-major mesh shards over its LAST axis, hence the order of the hybrid mesh."""

    DP = "dp"
    DP_REPLICATE = "dp_replicate"
    DP_SHARD = "dp_shard"
    TP = "tp"


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _must_span_world(dp_size: int, what: str) -> None:
    # init_device_mesh numbers ranks 0..n-1 without checking: ranks left out would fail with a bare IndexError while
    # the others block in the mesh's first collective
    if dp_size != _world():
        raise ValueError(f"a {what} must span the whole job: got {dp_size} ranks in a world of {_world()}; build a "
                         "sub-world mesh from its own process group (dp_group=...) instead")


def build_dp_mesh(dp_size: int, dp_replicate_size: int = 1, dp_group=None, device_type: str = "cuda") -> DeviceMesh:
    """The data-parallel mesh: ``(dp_replicate, dp_shard)`` when ``dp_replicate_size > 1`` (state is sharded inside a
    replica group and replicated across them), else ``(dp,)`` over ``dp_group`` or the whole job."""
    if dp_replicate_size > 1:
        if dp_group is not None:
            raise ValueError("dp_group describes a 1-D mesh and cannot be combined with dp_replicate_size > 1")
        if dp_size % dp_replicate_size:
            raise ValueError(f"dp_replicate_size ({dp_replicate_size}) must divide the data-parallel width ({dp_size})")
        _must_span_world(dp_size, "2-D hybrid-sharding mesh")
        return init_device_mesh(device_type, (dp_replicate_size, dp_size // dp_replicate_size),
                                mesh_dim_names=(MeshDim.DP_REPLICATE, MeshDim.DP_SHARD))
    if dp_group is not None:
        return DeviceMesh.from_group(dp_group, device_type, mesh_dim_names=(MeshDim.DP,))
    _must_span_world(dp_size, "1-D data-parallel mesh")
    return init_device_mesh(device_type, (dp_size,), mesh_dim_names=(MeshDim.DP,))


def build_dp_tp_mesh(tp_size: int, dp_size: int = 1, device_type: str = "cuda") -> DeviceMesh:
    """``(tp,)`` when there is no data parallelism, else row-major ``(dp, tp)``: consecutive ranks share a row, which is
    also how the entry points cut tensor-parallel blocks."""
    if dp_size == 1:
        return init_device_mesh(device_type, (tp_size,), mesh_dim_names=(MeshDim.TP,))
    return init_device_mesh(device_type, (dp_size, tp_size), mesh_dim_names=(MeshDim.DP, MeshDim.TP))


def mesh_dim_names(mesh: DeviceMesh | None) -> tuple[str, ...]:
    return tuple(getattr(mesh, "mesh_dim_names", None) or ())


def axis_group(mesh: DeviceMesh | None, name: str):
    """Process group of a named axis, or None when the mesh has no such axis."""
    if mesh is None or name not in mesh_dim_names(mesh):
        return None
    return mesh[name].get_group() if len(mesh_dim_names(mesh)) > 1 else mesh.get_group()


def tp_group(mesh: DeviceMesh | None):
    """The tensor-parallel group; an unnamed mesh is taken to be a bare tensor-parallel mesh."""
    if mesh is not None and not mesh_dim_names(mesh):
        return mesh.get_group()
    return axis_group(mesh, MeshDim.TP)


def dp_group(mesh: DeviceMesh | None):
    return axis_group(mesh, MeshDim.DP)


def shard_and_replicate_groups(mesh: DeviceMesh | None):
    """``(shard group, replicate group)`` of a data-parallel mesh: the group optimizer state is cut over, and the group
    whose members hold copies of the same slice (None without hybrid sharding)."""
    names = mesh_dim_names(mesh)
    if MeshDim.DP_SHARD in names:
        return axis_group(mesh, MeshDim.DP_SHARD), axis_group(mesh, MeshDim.DP_REPLICATE)
    return dp_group(mesh), None


# ---- DTensor views ----------------------------------------------------------------------------------------------------
def as_dtensor(local: torch.Tensor, mesh: DeviceMesh, shard_dim: int | None = 0, axis: str | None = None):
    """Wrap a locally held shard as a ``DTensor``: sharded along ``shard_dim`` over ``axis`` (default: the mesh's last
    axis) and replicated over every other axis; ``shard_dim=None`` means replicated everywhere. Shards must be even
    (the framework's slices are)."""
    from torch.distributed.tensor import DTensor, Replicate, Shard

    names = mesh_dim_names(mesh)
    axis = axis or (names[-1] if names else None)
    placements = []
    for i in range(mesh.ndim):
        name = names[i] if names else None
        placements.append(Shard(shard_dim) if shard_dim is not None and (name == axis or not names) else Replicate())
    return DTensor.from_local(local, mesh, placements, run_check=False)


def to_local(t):
    """The local shard of a ``DTensor``; plain tensors pass through (the role of the reference's DTensor access helpers)."""
    return t.to_local() if hasattr(t, "to_local") else t


def full_tensor(t):
    """The whole tensor of a ``DTensor`` (a collective gather over its sharded axes); plain tensors pass through."""
    return t.full_tensor() if hasattr(t, "full_tensor") else t


def expert_bank_dtensor(bank: torch.Tensor, ep_group, device_type: str | None = None):
    """An expert bank ``[E_local, ...]`` held by one expert-parallel rank as a DTensor sharded over experts."""
    mesh = DeviceMesh.from_group(ep_group, device_type or bank.device.type, mesh_dim_names=("ep",))
    return as_dtensor(bank, mesh, 0, "ep")
