"""Typed tuning surface of the fused TriMul.

Keeps the vocabulary of the reference's ``fold_cp_ops/distributed/workflows/trimul_tuning.py:72-217``
-- ``TriMulTuning`` holding a ``FrontTuning``, ``BackTuning``, ``OutGateTuning`` and
``TransportTuning``, every knob ``None`` until set, ``TriMulTuning().to_engine_kwargs() == {}`` -- so
call sites written against it keep working, and adds the choices the sm_100a kernels really have:

    BackTuning.contract_form        "auto" | "single" | "pair": one CTA per 128 x 256 tile of the
                                    contraction, or a CTA pair (tcgen05 cta_group::2) per 256 x 256 tile
    FrontTuning.fixed_order         True: every CTA of the projection kernel walks its gated chunks in
                                    the same order (default: rotated, which spreads the peer stores)
    TransportTuning.wait_timeout_ms bound of the cross-rank flag waits

The reference's remaining knobs pick SM90 tile shapes, cluster widths and NVSHMEM drains.  They are
still accepted and reach the engine under the engine's own spelling, where they change nothing
(``IGNORED_ON_SM100``).  ``engine.SM100_DEFAULTS`` holds the measured default per (feature width, cp).

How a knob is declared: ``_knob("engine_keyword")`` is a dataclass field defaulting to ``None`` whose
metadata carries the engine's keyword; ``_tuning_group`` freezes the class and derives its
``_ENGINE_KEYS`` table from that metadata, so a field and its keyword cannot drift apart.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Iterator, Optional, Tuple

__all__ = ["TriMulTuning", "FrontTuning", "BackTuning", "OutGateTuning", "TransportTuning", "NOT_EXPOSED",
           "IGNORED_ON_SM100"]


def _knob(engine_keyword: str):
    return dataclasses.field(default=None, metadata={"engine_keyword": engine_keyword})


def _tuning_group(cls):
    """Freeze ``cls`` as a dataclass and publish ``cls._ENGINE_KEYS`` = {field name: engine keyword}."""
    cls = dataclasses.dataclass(frozen=True)(cls)
    cls._ENGINE_KEYS = {f.name: f.metadata["engine_keyword"] for f in dataclasses.fields(cls)
                        if "engine_keyword" in f.metadata}
    return cls


def _set_knobs(group) -> Iterator[Tuple[str, Any]]:
    """(engine keyword, value) of every knob of ``group`` that is not ``None``."""
    for name, keyword in type(group)._ENGINE_KEYS.items():
        value = getattr(group, name)
        if value is not None:
            yield keyword, value


@_tuning_group
class FrontTuning:
    """The gated projection kernel and the front reshard it carries."""
    tile_mn: Optional[Tuple[int, int]] = _knob("front_tile_mn")
    pad_inner: Optional[bool] = _knob("front_pad_inner")
    pad_eager: Optional[bool] = _knob("front_pad_eager")
    fixed_order: Optional[bool] = _knob("front_fixed_order")


@_tuning_group
class BackTuning:
    """The triangle contraction kernel and the back reshard it carries."""
    tile_mn: Optional[Tuple[int, int]] = _knob("back_tile_mn")
    pingpong: Optional[bool] = _knob("back_pingpong")
    cluster_n: Optional[int] = _knob("back_cluster_n")
    contract_form: Optional[str] = _knob("contract_form")
    band_rows: Optional[int] = _knob("contract_band_rows")
    fixed_start: Optional[bool] = _knob("contract_fixed_start")
    pace_ns: Optional[int] = _knob("contract_pace_ns")


@_tuning_group
class OutGateTuning:
    """The output LayerNorm + gated output projection."""
    consumer: Optional[str] = _knob("consumer")


@_tuning_group
class TransportTuning:
    """How ranks learn that a reshard has landed."""
    device_signal_nvlink: Optional[bool] = _knob("use_device_signal_nvlink")
    wait_timeout_ms: Optional[float] = _knob("wait_timeout_ms")


@_tuning_group
class TriMulTuning:
    """Everything tunable about one fused TriMul module; changes nothing until a knob is set."""
    front: FrontTuning = dataclasses.field(default_factory=FrontTuning)
    back: BackTuning = dataclasses.field(default_factory=BackTuning)
    out_gate: OutGateTuning = dataclasses.field(default_factory=OutGateTuning)
    transport: TransportTuning = dataclasses.field(default_factory=TransportTuning)
    autotune: Optional[bool] = _knob("autotune_config")
    persistent: Optional[bool] = _knob("is_persistent")

    def to_engine_kwargs(self) -> Dict[str, Any]:
        """The set knobs as engine constructor keywords; an untouched tuning gives ``{}``."""
        flat: Dict[str, Any] = {}
        for group in (self.front, self.back, self.out_gate, self.transport, self):
            flat.update(_set_knobs(group))
        return flat


#: engine keywords kept for call sites written against the SM90 engine; the sm_100a kernels have no
#: such choice and ignore them
IGNORED_ON_SM100 = ("front_tile_mn", "front_pad_inner", "front_pad_eager", "back_tile_mn", "back_pingpong",
                    "back_cluster_n", "consumer", "use_device_signal_nvlink", "autotune_config", "is_persistent")

#: engine constructor keywords that are deliberately NOT tuning knobs, each with the reason
NOT_EXPOSED = {
    "device_mesh": "where the ranks are: the module's constructor argument, not a speed",
    "placements": "how the tensor is sharded: the module's constructor argument, not a speed",
    "dynamic": "only True exists: one engine serves every token extent",
    "has_mask": "decided by whether the call passes a mask",
    "eps": "a hyperparameter of the model, passed by name to the module",
    "composite_k": "names the incoming receive layout on a 1-D shard; follows from (direction, cp1)",
    "route2_ni": "names the incoming receive layout on a 2-D shard; follows from (direction, cp1)",
    "allocate": "whether the constructor allocates its buffers at once; a lifetime choice, not a speed",
}
