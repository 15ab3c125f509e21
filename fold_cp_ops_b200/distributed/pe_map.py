"""(DeviceMesh, placements) -> flat cp peer index -> global rank.

Public surface of the reference's ``fold_cp_ops/distributed/pe_map.py:113-306``: a ``PeMap``
dataclass built by :meth:`PeMap.from_mesh_placements`.  The cp (communication) axes are the mesh
dims whose placement is a ``Shard``; they are flattened row-major in mesh-dim order into one peer
index ``r in [0, cp)``, and ``cp_pe_table[r]`` is the global rank of peer ``r`` (dp coordinates
held at this rank's own position).  In this build the table indexes the per-peer symmetric-buffer
pointers the kernels store through, instead of NVSHMEM PE numbers; the ordering contract is the
same.  Everything here is host-side and needs no GPU: the mesh rank tensor is searched offline.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from .layout_map import LayoutRightMap

__all__ = ["PeMap"]


def _is_shard(placement) -> bool:
    """Duck-typed ``Shard`` test (works on DTensor placements and on simple stand-ins)."""
    probe = getattr(placement, "is_shard", None)
    if callable(probe):
        return bool(probe())
    return isinstance(getattr(placement, "dim", None), int)


def _placement_shard_dim(placement) -> Optional[int]:
    return getattr(placement, "dim", None) if _is_shard(placement) else None


def _mesh_rank_tensor(device_mesh) -> np.ndarray:
    mesh = device_mesh.mesh
    if isinstance(mesh, torch.Tensor):
        return mesh.detach().cpu().numpy()
    return np.asarray(mesh)


@dataclass
class PeMap:
    """Flat cp peer ordering for one rank.

    Attributes: ``cp`` peers; ``my_cp_rank`` this rank's own index; ``cp_pe_table`` int32 ``(cp,)``
    global rank per peer; ``cp_axes`` the sharded mesh dims; ``cp_axis_sizes`` their sizes
    (product = cp); ``cp_shard_tensor_dims`` the tensor dim each shards; ``device`` of the table.
    """

    cp: int
    my_cp_rank: int
    cp_pe_table: torch.Tensor
    cp_axes: Tuple[int, ...]
    cp_axis_sizes: Tuple[int, ...]
    cp_shard_tensor_dims: Tuple[int, ...]
    device: torch.device

    @property
    def cp_layout_shape_stride(self):
        """``((cp,), (1,))``: shape and stride of the 1-D peer table."""
        return ((self.cp,), (1,))

    def __repr__(self) -> str:
        return (f"PeMap(cp={self.cp}, my_cp_rank={self.my_cp_rank}, cp_axes={self.cp_axes}, "
                f"cp_axis_sizes={self.cp_axis_sizes}, cp_shard_tensor_dims={self.cp_shard_tensor_dims}, "
                f"cp_pe_table={self.cp_pe_table.tolist()}, device={self.device})")

    @staticmethod
    def from_mesh_placements(device_mesh, placements: Sequence, *, my_rank: Optional[int] = None,
                             device: Optional[torch.device] = None, distributed_manager=None) -> "PeMap":
        """Build the map.  ``distributed_manager`` only supplies defaults for rank and device.

        Raises ``ValueError`` when ``len(placements) != mesh.ndim``, when no axis is sharded,
        when ``my_rank`` does not appear exactly once in the mesh, or is missing from its own
        cp group.
        """
        ranks = _mesh_rank_tensor(device_mesh)
        if len(placements) != ranks.ndim:
            raise ValueError(f"placements length {len(placements)} != device_mesh ndim {ranks.ndim} "
                             f"(mesh shape {ranks.shape})")
        cp_axes = tuple(ax for ax, p in enumerate(placements) if _is_shard(p))
        if not cp_axes:
            raise ValueError(f"No sharded mesh axis found in placements {placements}; the cp all-to-all needs "
                             "at least one Shard axis (the token sharding).")
        cp_axis_sizes = tuple(int(ranks.shape[ax]) for ax in cp_axes)
        shard_dims = tuple(int(_placement_shard_dim(placements[ax])) for ax in cp_axes)
        cp = int(np.prod(cp_axis_sizes))

        if my_rank is None:
            if distributed_manager is not None:
                my_rank = int(distributed_manager.rank)
            elif torch.distributed.is_available() and torch.distributed.is_initialized():
                my_rank = int(torch.distributed.get_rank())
            else:
                my_rank = 0
        hits = np.argwhere(ranks == my_rank)
        if hits.shape[0] != 1:
            raise ValueError(f"rank {my_rank} appears {hits.shape[0]} times in the mesh rank tensor "
                             f"(expected exactly 1); mesh shape {ranks.shape}")
        here = [int(c) for c in hits[0]]

        flat = LayoutRightMap(cp_axis_sizes)
        table = np.empty(cp, dtype=np.int64)
        mine = -1
        for r in range(cp):
            coord = list(here)
            for ax, c in zip(cp_axes, flat.unravel(r)):
                coord[ax] = int(c)
            table[r] = int(ranks[tuple(coord)])
            if table[r] == my_rank:
                mine = r
        if mine < 0:
            raise ValueError(f"this rank {my_rank} not found in its own cp group {table.tolist()}")

        if device is None:
            dm_dev = getattr(distributed_manager, "device", None) if distributed_manager is not None else None
            if dm_dev is not None:
                device = dm_dev
            elif torch.cuda.is_available():
                device = torch.device("cuda", torch.cuda.current_device())
            else:
                device = torch.device("cpu")
        device = torch.device(device)
        return PeMap(cp=cp, my_cp_rank=mine, cp_pe_table=torch.tensor(table, dtype=torch.int32, device=device),
                     cp_axes=cp_axes, cp_axis_sizes=cp_axis_sizes, cp_shard_tensor_dims=shard_dims, device=device)
