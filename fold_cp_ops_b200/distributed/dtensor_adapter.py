"""DTensor duck-typing and TriMul sharding validation.

Mirrors ``fold_cp_ops/distributed/dtensor_adapter.py:108-269`` of the reference: the feature dim
(3) must stay whole on every rank (both LayerNorms and the projections reduce over it), at least
one token dim (1 or 2) must be sharded, ``Shard(0)`` on the batch is a passthrough, and a
``Shard`` on a size-1 mesh axis is treated as ``Replicate``.
"""
from __future__ import annotations

from typing import Sequence, Tuple

from .pe_map import _is_shard, _placement_shard_dim

_TOKEN_TENSOR_DIMS = (1, 2)


def _is_dtensor(x) -> bool:
    return hasattr(x, "to_local") and hasattr(x, "_spec") and hasattr(x, "device_mesh")


def _dtensor_mesh_placements(x):
    """``(device_mesh, placements)`` of a DTensor, with the ``_spec`` fallback."""
    spec = getattr(x, "_spec", None)
    found = []
    for own, from_spec in (("device_mesh", "mesh"), ("placements", "placements")):
        value = getattr(x, own, None)
        found.append(getattr(spec, from_spec) if value is None and spec is not None else value)
    return found[0], tuple(found[1])


def _rowmaj_stride(shape: Sequence[int]) -> Tuple[int, ...]:
    stride, acc = [], 1
    for n in reversed(tuple(shape)):
        stride.append(acc)
        acc *= int(n)
    return tuple(reversed(stride))


def _shards(placements: Sequence):
    """``(mesh axis, tensor dim)`` of every ``Shard`` placement, in mesh-axis order."""
    return [(axis, _placement_shard_dim(p)) for axis, p in enumerate(placements) if _is_shard(p)]


def _split_of_tensor_dim(device_mesh, placements: Sequence, tensor_dim: int) -> int:
    """How many ways the mesh splits ``tensor_dim`` (product of the sizes of the axes that shard it)."""
    sizes = tuple(device_mesh.mesh.shape)
    ways = 1
    for axis, dim in _shards(placements):
        if dim == tensor_dim:
            ways *= int(sizes[axis])
    return ways


def validate_trimul_sharding(placements: Sequence, ndim_mesh: int) -> Tuple[int, ...]:
    """Return the mesh dims that shard a token axis; raise ``ValueError`` on an unusable sharding."""
    if len(placements) != ndim_mesh:
        raise ValueError(f"placements length {len(placements)} != mesh ndim {ndim_mesh}")
    shards = _shards(placements)
    if any(dim == 3 for _, dim in shards):
        raise ValueError("TriMul requires the feature dim (3) to be UN-sharded (LN + DualGatedGEMM reduce over "
                         f"full D), but placements {placements} shard tensor dim 3.")
    token_axes = tuple(axis for axis, dim in shards if dim in _TOKEN_TENSOR_DIMS)
    if not token_axes:
        raise ValueError("TriMul requires at least one token axis (tensor dim 1 or 2) to be sharded over the cp "
                         f"mesh, but placements {placements} shard none. Expected the "
                         "(Shard(0),Shard(1),Shard(2)) pattern.")
    return token_axes


def _token_split_factor(device_mesh, placements: Sequence) -> int:
    """Product of the mesh-axis sizes that split a token axis; 1 means the contraction is local."""
    rows, cols = (_split_of_tensor_dim(device_mesh, placements, dim) for dim in _TOKEN_TENSOR_DIMS)
    return rows * cols


def _effective_placements(device_mesh, placements: Sequence) -> list:
    """Placements with every ``Shard`` on a size-1 mesh axis replaced by ``Replicate``."""
    from torch.distributed.tensor import Replicate

    shape = tuple(device_mesh.mesh.shape)
    return [Replicate() if (_is_shard(p) and int(shape[axis]) == 1) else p for axis, p in enumerate(placements)]


def _ensure_nvshmem(distributed_manager=None) -> None:
    """Bring up the symmetric-memory runtime for the cp reshards (idempotent, collective).

    The name is the reference's; here it initialises the peer-memory plumbing
    ``DistributedManager.init_nvshmem`` owns (torch symmetric memory over NVLink)."""
    manager_cls = type(distributed_manager) if distributed_manager is not None else None
    if manager_cls is None or not hasattr(manager_cls, "init_nvshmem"):
        from .distributed_manager import DistributedManager as manager_cls
    manager_cls.init_nvshmem()


def _is_rows_sharded_canonical(device_mesh, placements: Sequence) -> bool:
    """True when the ONLY token axis split over the mesh is the row axis (tensor dim 1): the
    canonical 1-D layout ``(dp=1, cp0=cp, cp1=1)``."""
    rows, cols = (_split_of_tensor_dim(device_mesh, placements, dim) for dim in _TOKEN_TENSOR_DIMS)
    return rows > 1 and cols == 1
