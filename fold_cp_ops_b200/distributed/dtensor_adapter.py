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
    mesh = getattr(x, "device_mesh", None)
    placements = getattr(x, "placements", None)
    spec = getattr(x, "_spec", None)
    if mesh is None and spec is not None:
        mesh = spec.mesh
    if placements is None and spec is not None:
        placements = spec.placements
    return mesh, tuple(placements)


def _rowmaj_stride(shape: Sequence[int]) -> Tuple[int, ...]:
    stride, acc = [], 1
    for n in reversed(tuple(shape)):
        stride.append(acc)
        acc *= int(n)
    return tuple(reversed(stride))


def validate_trimul_sharding(placements: Sequence, ndim_mesh: int) -> Tuple[int, ...]:
    """Return the mesh dims that shard a token axis; raise ``ValueError`` on an unusable sharding."""
    if len(placements) != ndim_mesh:
        raise ValueError(f"placements length {len(placements)} != mesh ndim {ndim_mesh}")
    sharded_dims, cp_axes = [], []
    for axis, p in enumerate(placements):
        if _is_shard(p):
            tdim = _placement_shard_dim(p)
            sharded_dims.append(tdim)
            if tdim in _TOKEN_TENSOR_DIMS:
                cp_axes.append(axis)
    if 3 in sharded_dims:
        raise ValueError("TriMul requires the feature dim (3) to be UN-sharded (LN + DualGatedGEMM reduce over "
                         f"full D), but placements {placements} shard tensor dim 3.")
    if not cp_axes:
        raise ValueError("TriMul requires at least one token axis (tensor dim 1 or 2) to be sharded over the cp "
                         f"mesh, but placements {placements} shard none. Expected the "
                         "(Shard(0),Shard(1),Shard(2)) pattern.")
    return tuple(cp_axes)


def _token_split_factor(device_mesh, placements: Sequence) -> int:
    """Product of the mesh-axis sizes that split a token axis; 1 means the contraction is local."""
    shape = tuple(device_mesh.mesh.shape)
    factor = 1
    for axis, p in enumerate(placements):
        if _is_shard(p) and _placement_shard_dim(p) in _TOKEN_TENSOR_DIMS:
            factor *= int(shape[axis])
    return factor


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
    shape = tuple(device_mesh.mesh.shape)
    rows = cols = 1
    for axis, p in enumerate(placements):
        if _is_shard(p):
            d = _placement_shard_dim(p)
            if d == 1:
                rows *= int(shape[axis])
            elif d == 2:
                cols *= int(shape[axis])
    return rows > 1 and cols == 1
