"""Typed tuning knobs for the fused TriMul, kept for call-site compatibility.

Same types and field names as the reference's
``fold_cp_ops/distributed/workflows/trimul_tuning.py:72-217``: ``TriMulTuning`` nests
``FrontTuning`` / ``BackTuning`` / ``OutGateTuning`` / ``TransportTuning``; every field defaults to
``None`` and ``TriMulTuning().to_engine_kwargs() == {}``.  The reference's knobs select SM90 tile
shapes, cluster widths and NVSHMEM drains; the sm_100a kernels have one fixed configuration per
feature width, so the engine accepts the flattened keywords and ignores the SM90-only ones
(listed in ``IGNORED_ON_SM100``).
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, Optional, Tuple

__all__ = ["TriMulTuning", "FrontTuning", "BackTuning", "OutGateTuning", "TransportTuning", "NOT_EXPOSED",
           "IGNORED_ON_SM100"]


@dataclass(frozen=True)
class FrontTuning:
    """Stage 2 (gated projection + front reshard)."""
    tile_mn: Optional[Tuple[int, int]] = None
    pad_inner: Optional[bool] = None
    pad_eager: Optional[bool] = None
    _ENGINE_KEYS = {"tile_mn": "front_tile_mn", "pad_inner": "front_pad_inner", "pad_eager": "front_pad_eager"}


@dataclass(frozen=True)
class BackTuning:
    """Stage 3 (triangle contraction + back reshard)."""
    tile_mn: Optional[Tuple[int, int]] = None
    pingpong: Optional[bool] = None
    cluster_n: Optional[int] = None
    _ENGINE_KEYS = {"tile_mn": "back_tile_mn", "pingpong": "back_pingpong", "cluster_n": "back_cluster_n"}


@dataclass(frozen=True)
class OutGateTuning:
    """Stage 4 (output LayerNorm + gated output projection)."""
    consumer: Optional[str] = None
    _ENGINE_KEYS = {"consumer": "consumer"}


@dataclass(frozen=True)
class TransportTuning:
    """Completion signalling of the two reshards."""
    device_signal_nvlink: Optional[bool] = None
    _ENGINE_KEYS = {"device_signal_nvlink": "use_device_signal_nvlink"}


@dataclass(frozen=True)
class TriMulTuning:
    """The whole surface; inert by default."""
    front: FrontTuning = field(default_factory=FrontTuning)
    back: BackTuning = field(default_factory=BackTuning)
    out_gate: OutGateTuning = field(default_factory=OutGateTuning)
    transport: TransportTuning = field(default_factory=TransportTuning)
    autotune: Optional[bool] = None
    persistent: Optional[bool] = None
    _ENGINE_KEYS = {"autotune": "autotune_config", "persistent": "is_persistent"}

    def to_engine_kwargs(self) -> Dict[str, Any]:
        """Flatten to engine keyword names, omitting every unset field (``{}`` when nothing is set)."""
        out: Dict[str, Any] = {}
        for group in (self.front, self.back, self.out_gate, self.transport):
            for f in fields(group):
                v = getattr(group, f.name)
                if v is not None:
                    out[type(group)._ENGINE_KEYS[f.name]] = v
        for name, key in TriMulTuning._ENGINE_KEYS.items():
            v = getattr(self, name)
            if v is not None:
                out[key] = v
        return out


#: engine keywords that exist for call-site compatibility and change nothing on sm_100a
IGNORED_ON_SM100 = ("front_tile_mn", "front_pad_inner", "front_pad_eager", "back_tile_mn", "back_pingpong",
                    "back_cluster_n", "consumer", "use_device_signal_nvlink", "autotune_config", "is_persistent")

#: engine parameters deliberately not reachable through the tuning surface, with the reason
NOT_EXPOSED = {
    "back_store": "one store design exists: the contraction epilogue writes to the token owner",
    "hybrid_ib": "single NVSwitch domain only; there is no InfiniBand transport",
    "route2_ni": "derived from (direction, cp1) -- a receive layout, not a speed",
    "composite_k": "derived from (direction, cp1) -- a receive layout, not a speed",
    "dynamic": "one supported value",
    "has_mask": "a property of the call, not a tuning choice",
    "eps": "a model hyperparameter, promoted to a named constructor argument",
    "front_pingpong": "the projection kernel has one schedule",
    "device_mesh": "topology, taken from the constructor",
    "placements": "topology, taken from the constructor",
}
