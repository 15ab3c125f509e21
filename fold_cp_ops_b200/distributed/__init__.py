"""Multi-GPU infrastructure of the fused TriMul (process group, cp mesh, peer map, symmetric
buffers, group-uniform guards).  Re-exports the same names as the reference's
``fold_cp_ops/distributed/__init__.py:35-65`` and nothing else; kernels are not imported here."""
from .collective_symmetry import BarrierTimeout, CollectiveError, CollectiveFailure, CollectiveGate, PeerFailure
from .distributed_manager import DistributedManager
from .layout_map import LayoutLeftMap, LayoutMap, LayoutRightMap
from .pe_map import PeMap
from .trimul_weights import W_KEYS, W_PROJ_BIAS_KEYS, weights_from_trimul_module

__all__ = [
    "BarrierTimeout",
    "CollectiveError",
    "CollectiveFailure",
    "CollectiveGate",
    "DistributedManager",
    "LayoutLeftMap",
    "LayoutMap",
    "LayoutRightMap",
    "PeMap",
    "PeerFailure",
    "W_KEYS",
    "W_PROJ_BIAS_KEYS",
    "weights_from_trimul_module",
]
