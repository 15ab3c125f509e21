"""The DTensor front door of the fused context-parallel TriMul.

Drop-in for the public surface of the reference's
``fold_cp_ops/distributed/workflows/trimul_autotuned.py:3806-4699``: exactly two public names,
``TriangularMultiplication`` (nn.Module, DTensor in -> DTensor out, cp=1 auto-selection,
outgoing / incoming) and the functional ``trimul_a2a``.  Construction resolves placements, cp
and the peer map and touches no GPU memory; ``prepare`` (or the first ``forward``) allocates the
symmetric operand buffers; ``forward`` checks mesh / placements / feature width, picks the
``(batch, masked)`` engine and re-wraps the local result with the input's own sharding.

The engine underneath (``TriMulAutotuned`` here, as there) is three sm_100a kernels whose
epilogues store straight into the owning peer's buffer; see :mod:`fold_cp_ops_b200.engine`.

Beyond the reference's surface the module offers ``check()`` (raise if a device-side wait of an
earlier forward expired) and ``last_forward_stats()`` (kernel times, time spent in the cross-rank
waits, bytes pushed to peers).
"""
from __future__ import annotations

import difflib
import inspect
import warnings
from typing import Dict, List, NamedTuple, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn

from ...engine import CpGeometry, TriMulEngine
from ...workflows.trimul_autotune import trimul_autotuned
from ..dtensor_adapter import (_dtensor_mesh_placements, _effective_placements, _ensure_nvshmem, _is_dtensor,
                               _rowmaj_stride, _token_split_factor, validate_trimul_sharding)
from ..pe_map import PeMap, _is_shard, _mesh_rank_tensor, _placement_shard_dim
from ..trimul_weights import W_KEYS, W_PROJ_BIAS_KEYS
from .trimul_tuning import IGNORED_ON_SM100, TriMulTuning  # noqa: F401  (re-exported for callers that import it here)

__all__ = ["TriangularMultiplication", "trimul_a2a"]

DIRECTIONS = ("outgoing", "incoming")
_LN_PARAM_KEYS = ("norm_in_w", "norm_in_b", "norm_out_w", "norm_out_b")
_WEIGHT_KEYS = tuple(W_KEYS) + tuple(W_PROJ_BIAS_KEYS)

#: receive layouts of the reference's incoming path.  This build always writes the transposed operand
#: plane for "incoming"; the names are reported so that callers which log them keep working.
INCOMING_STORE_VARIANTS = ("plain", "composite_k", "route2_ni")


def _weight_vocabulary_mismatch() -> str:
    """The single-GPU entry point takes every weight as a keyword.  Returns a description of any
    difference between those keywords and the 12-key weight dict ('' when they agree)."""
    not_weights = {"x", "mask", "direction", "eps", "out", "select", "_config"}
    accepted = set(inspect.signature(trimul_autotuned).parameters) - not_weights
    missing, extra = sorted(set(_WEIGHT_KEYS) - accepted), sorted(accepted - set(_WEIGHT_KEYS))
    if not missing and not extra:
        return ""
    return (f"weight dict keys {missing} are not keywords of trimul_autotuned; its keywords {extra} are not weight "
            "dict keys")


if _weight_vocabulary_mismatch():  # a packaging error, caught at import instead of at the first cp=1 forward
    raise ImportError(_weight_vocabulary_mismatch())


# ---------------------------------------------------------------------------------------------
# cp=1 routing and re-wrapping
# ---------------------------------------------------------------------------------------------
def _is_single_device(x) -> bool:
    """Whether ``x`` can be served by one GPU with no communication: anything that is not a DTensor,
    a DTensor on a mesh of one device, or a DTensor whose placements leave both token axes whole
    (for example a data-parallel mesh that only shards the batch)."""
    if not _is_dtensor(x):
        return True
    mesh, placements = _dtensor_mesh_placements(x)
    if mesh is None:
        return True
    devices = int(mesh.mesh.numel())
    return devices == 1 or _token_split_factor(mesh, _effective_placements(mesh, placements)) <= 1


def _rewrap_like(x, out_local):
    """Give ``out_local`` the distributed identity of ``x`` (mesh, placements, global shape and
    row-major stride); a plain tensor input gets the plain tensor back."""
    if not _is_dtensor(x):
        return out_local
    from torch.distributed.tensor import DTensor

    mesh, placements = _dtensor_mesh_placements(x)
    global_shape = torch.Size(tuple(x.shape))
    return DTensor.from_local(out_local, mesh, list(placements), shape=global_shape,
                              stride=_rowmaj_stride(tuple(global_shape)), run_check=False)


def _local(t):
    return t.to_local() if _is_dtensor(t) else t


def _trimul_single_device(x, w: dict, *, direction: str, mask, eps: float = 1e-5):
    """The cp=1 route: unwrap, run the single-GPU chain, wrap again."""
    strangers = sorted(set(w) - set(_WEIGHT_KEYS))
    if strangers:
        raise KeyError(f"cp=1 TriMul fallback got unexpected weight key(s) {strangers}; "
                       f"expected exactly {list(_WEIGHT_KEYS)}")
    kwargs = {}
    for key in _WEIGHT_KEYS:
        t = w.get(key)
        kwargs[key] = t.float() if (t is not None and key in _LN_PARAM_KEYS) else t
    out_local = trimul_autotuned(_local(x), **kwargs, mask=_local(mask), direction=direction, eps=eps,
                                 select="heuristic")
    return _rewrap_like(x, out_local)


def incoming_store_variant(direction: str, cp1: int, batch: int = 1) -> str:
    """Name of the reference's front-store variant for a configuration -- a total function of
    ``(direction, cp1)``: outgoing is ``plain``; incoming is ``composite_k`` on a 1-D token shard
    (``cp1 == 1``) and ``route2_ni`` on a 2-D one.  ``batch`` only has to be a positive integer."""
    if direction not in DIRECTIONS:
        raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}. Falling through to "
                         "the plain store on a typo would silently cost ~2x on the incoming path.")
    for name, value in (("cp1", cp1), ("batch", batch)):
        if int(value) < 1:
            raise ValueError(f"{name} must be >= 1; got {value!r}")
    table = {("outgoing", False): "plain", ("outgoing", True): "plain",
             ("incoming", False): "composite_k", ("incoming", True): "route2_ni"}
    return table[(direction, int(cp1) > 1)]


# ---------------------------------------------------------------------------------------------
# geometry from (mesh, placements)
# ---------------------------------------------------------------------------------------------
def _token_placements(device_mesh, placements):
    """Effective placements with batch shards (``Shard(0)``: data parallel, no communication)
    replaced by ``Replicate`` so that only token axes remain as cp axes."""
    from torch.distributed.tensor import Replicate

    eff = _effective_placements(device_mesh, placements)
    return [Replicate() if (_is_shard(p) and _placement_shard_dim(p) == 0) else p for p in eff]


def _geometry_from_pe_map(pe_map: PeMap) -> CpGeometry:
    """Row-major (row block, column block) geometry the kernels use, from a :class:`PeMap`.

    The PeMap flattens the cp mesh axes in MESH order; the kernels order peers by
    (tensor dim 1 block, tensor dim 2 block).  The two agree unless the mesh lists the column
    axis first, in which case the peer table is permuted here."""
    dims = tuple(pe_map.cp_shard_tensor_dims)
    sizes = tuple(int(s) for s in pe_map.cp_axis_sizes)
    if any(d not in (1, 2) for d in dims) or len(set(dims)) != len(dims):
        raise ValueError(f"each cp mesh axis must shard a distinct token dim (1 or 2); got tensor dims {dims}")
    cp0 = sizes[dims.index(1)] if 1 in dims else 1
    cp1 = sizes[dims.index(2)] if 2 in dims else 1
    table = pe_map.cp_pe_table.tolist()

    def pemap_index(r0: int, r1: int) -> int:
        if len(dims) == 1:
            return r0 if dims[0] == 1 else r1
        return r0 * cp1 + r1 if dims == (1, 2) else r1 * cp0 + r0

    peers = tuple(int(table[pemap_index(r0, r1)]) for r0 in range(cp0) for r1 in range(cp1))
    me = int(table[pe_map.my_cp_rank])
    return CpGeometry(cp0=cp0, cp1=cp1, rank=peers.index(me), peers=peers)


_CP_GROUP_CACHE: dict = {}


def _resolve_cp_group(device_mesh, placements, geometry: CpGeometry):
    """The process group holding exactly this rank's cp peers.  COLLECTIVE when it has to create
    groups (a mesh with dp axes and a 2-D token split): every rank creates every cp group of the
    mesh in the same order."""
    import torch.distributed as dist

    peers = sorted(geometry.peers)
    if peers == list(range(dist.get_world_size())):
        return dist.group.WORLD
    token_axes = [ax for ax, p in enumerate(placements) if _is_shard(p) and _placement_shard_dim(p) in (1, 2)]
    if len(token_axes) == 1:
        return device_mesh.get_group(token_axes[0])
    ranks = _mesh_rank_tensor(device_mesh)
    other = [ax for ax in range(ranks.ndim) if ax not in token_axes]
    moved = np.moveaxis(ranks, other, list(range(len(other)))).reshape(-1, len(peers)) if other else ranks.reshape(1, -1)
    mine = None
    for row in moved:
        key = tuple(sorted(int(r) for r in row))
        grp = _CP_GROUP_CACHE.get(key)
        if grp is None:
            grp = dist.new_group(ranks=list(key))
            _CP_GROUP_CACHE[key] = grp
        if list(key) == peers:
            mine = grp
    if mine is None:
        raise RuntimeError(f"could not find a process group for cp peers {peers}")
    return mine


# ---------------------------------------------------------------------------------------------
# the engine, under the reference's name and constructor signature
# ---------------------------------------------------------------------------------------------
class TriMulAutotuned(TriMulEngine):
    """Fused cp TriMul engine for one ``(batch, masked)`` variant.

    Same constructor shape as the reference's ``TriMulAutotuned(pe_map, B, N, D, w, dt, **kw)``
    (``fold_cp_ops/distributed/workflows/trimul_autotuned.py:2686``).  ``B`` / ``N`` size the
    buffers allocated up front; any other ``N`` meeting the divisibility rules is served later
    (always dynamic).  ``contract_form``, ``contract_band_rows``, ``contract_fixed_start``, ``contract_pace_ns``, ``front_fixed_order`` and ``wait_timeout_ms`` are the
    sm_100a choices (see :class:`fold_cp_ops_b200.engine.TriMulEngine`); keywords that configured
    SM90 tiles or NVSHMEM drains are accepted and ignored (``trimul_tuning.IGNORED_ON_SM100``)."""

    def __init__(self, pe_map: PeMap, B: int, N: int, D: int, w: dict, dt: torch.dtype, *, device_mesh=None,
                 placements=None, dynamic: bool = True, has_mask: bool = False, eps: float = 1e-5,
                 composite_k: bool = False, route2_ni: bool = False, contract_form: Optional[str] = None,
                 front_fixed_order: Optional[bool] = None, contract_band_rows: Optional[int] = None,
                 contract_fixed_start: Optional[bool] = None, contract_pace_ns: Optional[int] = None,
                 wait_timeout_ms: Optional[float] = None, front_tile_mn=None, front_pad_inner=None, front_pad_eager=None, back_tile_mn=None,
                 back_pingpong=None, back_cluster_n=None, consumer=None, use_device_signal_nvlink=None,
                 autotune_config=None, is_persistent=None, allocate: bool = True):
        if dt is not torch.bfloat16:
            raise ValueError(f"the sm_100a TriMul kernels compute in torch.bfloat16; got dtype={dt}")
        if not dynamic:
            raise ValueError("dynamic=False is not supported: one engine serves every token extent")
        if int(w["norm_in_w"].shape[0]) != int(D):
            raise ValueError(f"D={D} disagrees with the weights' feature width {int(w['norm_in_w'].shape[0])}")
        geometry = _geometry_from_pe_map(pe_map)
        cp = geometry.cp
        if D % cp != 0:
            raise ValueError(f"D={D} must be divisible by cp={cp} (each rank contracts D/cp channels)")
        if N % geometry.cp0 != 0 or N % geometry.cp1 != 0:
            raise ValueError(f"N={N} must be divisible by each cp axis {(geometry.cp0, geometry.cp1)}")
        if N % 8 != 0:
            raise ValueError(f"N={N} must be a multiple of 8 (16-byte rows of bf16)")
        if (N // geometry.cp0) % 8 != 0 or (N // geometry.cp1) % 8 != 0:
            raise ValueError(f"local token extents {(N // geometry.cp0, N // geometry.cp1)} must be multiples of 8")
        group = None
        if cp > 1:
            if device_mesh is None or placements is None:
                raise ValueError("a cp > 1 engine needs device_mesh= and placements= to find its peers' process group")
            group = _resolve_cp_group(device_mesh, _token_placements(device_mesh, placements), geometry)
        super().__init__(w, device=pe_map.device, eps=eps, geometry=geometry, process_group=group,
                         contract_form=contract_form, front_fixed_order=front_fixed_order,
                         contract_band_rows=contract_band_rows, contract_fixed_start=contract_fixed_start,
                         contract_pace_ns=contract_pace_ns, wait_timeout_ms=wait_timeout_ms)
        self.pe_map = pe_map
        self.has_mask = bool(has_mask)
        self.composite_k = bool(composite_k)
        self.route2_ni = bool(route2_ni)
        self.dynamic = True
        if allocate:
            self.prepare(int(B), int(N))

    @property
    def store_variant(self) -> str:
        """Which of :data:`INCOMING_STORE_VARIANTS` this engine was asked for."""
        return "composite_k" if self.composite_k else ("route2_ni" if self.route2_ni else "plain")


def _engine_keywords() -> List[str]:
    """Keyword-only parameters of the engine constructor, i.e. what ``**fused_kwargs`` may contain."""
    params = inspect.signature(TriMulAutotuned.__init__).parameters.values()
    return sorted(p.name for p in params if p.kind is inspect.Parameter.KEYWORD_ONLY)


def _reject_unknown_engine_kwargs(fused_kwargs: dict) -> None:
    """A misspelt engine keyword must fail at the caller's own line, not later inside the lazily
    built engine.  Raises ``TypeError`` naming each stranger and its nearest legal spelling."""
    legal = _engine_keywords()
    complaints = []
    for name in sorted(fused_kwargs):
        if name in legal:
            continue
        close = difflib.get_close_matches(name, legal, n=1)
        complaints.append(f"{name!r} (did you mean {close[0]!r}?)" if close else f"{name!r}")
    if complaints:
        raise TypeError(f"trimul_a2a got unknown fused_kwargs: {', '.join(complaints)}. Legal engine knobs are {legal}. "
                        "Refused here rather than inside the lazy engine build, which happens after the PeMap and the "
                        "symmetric buffers are up and reports a TypeError from a constructor you did not call.")


class _EngineKey(NamedTuple):
    """What distinguishes two engines of the functional form's cache."""
    batch: int
    token_extent: Optional[int]   # None for a dynamic engine (serves every extent)
    width: int
    axis_sizes: Tuple[int, ...]
    masked: bool
    store_variant: str


def _store_variant_kwargs(kw: dict, direction: str, cp1: int, batch: int) -> dict:
    """``kw`` plus the store-variant flag of this configuration, unless the caller chose one."""
    if "composite_k" in kw or "route2_ni" in kw:
        return kw
    variant = incoming_store_variant(direction, cp1, batch)
    return kw if variant == "plain" else dict(kw, **{variant: True})


def _build_pe_map(x, distributed_manager):
    mesh, placements = _dtensor_mesh_placements(x)
    validate_trimul_sharding(placements, mesh.ndim)
    pe_map = PeMap.from_mesh_placements(mesh, _token_placements(mesh, placements),
                                        distributed_manager=distributed_manager)
    return pe_map, mesh, placements


def _get_engine(cache: dict, pe_map, mesh, placements, B, N, D, w, dt, *, dynamic, has_mask, kw,
                distributed_manager=None):
    variant = "composite_k" if kw.get("composite_k") else ("route2_ni" if kw.get("route2_ni") else "plain")
    key = _EngineKey(int(B), None if dynamic else int(N), int(D), tuple(int(s) for s in pe_map.cp_axis_sizes),
                     bool(has_mask), variant)
    eng = cache.get(key)
    if eng is None:
        _ensure_nvshmem(distributed_manager)
        eng = cache[key] = TriMulAutotuned(pe_map, int(B), int(N), int(D), w, dt, device_mesh=mesh,
                                           placements=placements, dynamic=dynamic, has_mask=has_mask, **kw)
    return eng


_FUSED_CACHE: dict = {}


def trimul_a2a(x, w: dict, dt: torch.dtype, *, direction: str = "outgoing", mask=None, dynamic: bool = True,
               distributed_manager=None, _cache: Optional[dict] = None, **fused_kwargs):
    """Functional form: DTensor ``(B, N, N, D)`` -> same-sharding DTensor.  Inference only.

    ``w`` is the replicated 12-key weight dict; ``mask`` a DTensor sharded like ``x``, a local
    tensor or ``None``.  cp == 1 inputs short-circuit to the single-GPU ``trimul_autotuned`` before
    any peer map is built.  ``_cache`` lets a caller own the engine cache; ``None`` uses a
    process-global one."""
    assert direction in DIRECTIONS, "direction must be 'outgoing'|'incoming'"
    _reject_unknown_engine_kwargs(fused_kwargs)
    if not isinstance(x, torch.Tensor) and not _is_dtensor(x):
        raise TypeError(f"trimul_a2a expects a DTensor or local Tensor x, got {type(x)}.")
    if _is_single_device(x):
        return _trimul_single_device(x, w, direction=direction, mask=mask, eps=fused_kwargs.get("eps", 1e-5))
    pe_map, mesh, placements = _build_pe_map(x, distributed_manager)
    B, N, _, D = (int(s) for s in x.shape)
    axis_sizes = tuple(int(s) for s in pe_map.cp_axis_sizes)
    kw = _store_variant_kwargs(dict(fused_kwargs), direction, axis_sizes[1] if len(axis_sizes) > 1 else 1, B)
    eng = _get_engine(_FUSED_CACHE if _cache is None else _cache, pe_map, mesh, placements, B, N, D, w, dt,
                      dynamic=dynamic, has_mask=mask is not None, kw=kw, distributed_manager=distributed_manager)
    return _rewrap_like(x, eng.forward(_local(x), direction, mask_local=_local(mask)))


# ---------------------------------------------------------------------------------------------
# nn.Module front door
# ---------------------------------------------------------------------------------------------
class TriangularMultiplication(nn.Module):
    """DTensor-in / DTensor-out inference drop-in for a context-parallel TriMul layer.

    Args:
        layer: any module exposing ``norm_in, p_in, g_in, norm_out, p_out, g_out``; weights are
            read ONCE here (all six biases are carried).  Missing submodule -> ``AttributeError``.
        direction: ``"outgoing"`` | ``"incoming"`` (anything else raises ``ValueError``).
        device_mesh: the mesh the layer is sharded over; recorded and CHECKED against the input of
            ``forward``, never dispatched on.  ``None`` for a cp=1 module.
        distributed_manager: live ``DistributedManager`` (needed for cp > 1 only).
        placements: per-mesh-dim placements; default ``[Shard(i + 1) for i in range(mesh.ndim)]``.
        dtype: compute dtype of the fused kernels (bf16).
        eps: LayerNorm epsilon; ``None`` takes ``layer.norm_in.eps`` (fallback 1e-5).
        tuning: optional :class:`TriMulTuning`; a default-constructed one equals ``None``.
    """

    _SUBMODULES = ("norm_in", "p_in", "g_in", "norm_out", "p_out", "g_out")

    def __init__(self, layer: nn.Module, direction: str, device_mesh, distributed_manager, *, placements=None,
                 dtype: torch.dtype = torch.bfloat16, eps: Optional[float] = None,
                 tuning: Optional[TriMulTuning] = None):
        super().__init__()
        if direction not in DIRECTIONS:
            raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}. It selects the "
                             "back-half einsum, so an unrecognised value would compute a different contraction.")
        from ..trimul_weights import weights_from_trimul_module

        weights = weights_from_trimul_module(layer)
        for key in _LN_PARAM_KEYS:  # the kernels read LayerNorm parameters as fp32
            if weights[key] is not None:
                weights[key] = weights[key].to(torch.float32)
        if eps is None:
            eps = getattr(getattr(layer, "norm_in", None), "eps", 1e-5)
        self._w, self._dt, self._dir, self._dm = weights, dtype, direction, distributed_manager
        self._eps = float(eps)
        self._tuning = tuning
        self._kw = {} if tuning is None else tuning.to_engine_kwargs()
        self.device_mesh = device_mesh
        self.direction = direction
        self._D = int(weights["norm_in_w"].shape[0])
        self._placements = self._resolve_placements(device_mesh, placements)
        self._cp, self._cp_axis_sizes, self._pe_map = self._resolve_cp(device_mesh, self._placements)
        self._cp1 = int(self._cp_axis_sizes[1]) if len(self._cp_axis_sizes) > 1 else 1
        self._engines: Dict[Tuple[int, bool], TriMulAutotuned] = {}
        self._engine_variant: Dict[Tuple[int, bool], str] = {}
        self._warned_second_variant = False
        for name in self._SUBMODULES:  # the layer's own submodules stay reachable (and in state_dict)
            setattr(self, name, getattr(layer, name))

    # -- construction helpers ------------------------------------------------------------------
    @staticmethod
    def _resolve_placements(device_mesh, placements):
        """One placement per mesh dim: the caller's, or ``Shard(1)[, Shard(2)]`` for a 1-D / 2-D mesh."""
        given = None if placements is None else list(placements)
        if device_mesh is None:
            return given
        if not (hasattr(device_mesh, "ndim") and hasattr(device_mesh, "mesh")):
            raise TypeError(f"device_mesh must be a DeviceMesh (it needs .ndim and .mesh) or None; got "
                            f"{type(device_mesh).__name__}. The constructor derives cp, the placements and the "
                            "PeMap from it, so an object that only compares equal is not enough.")
        ndim = int(device_mesh.ndim)
        if given is not None:
            if len(given) != ndim:
                raise ValueError(f"placements has {len(given)} entries but device_mesh.ndim is {ndim}. One placement "
                                 "per mesh dim is required; there is no padding rule.")
            return given
        if ndim > 2:
            raise ValueError(f"TriangularMultiplication cannot default the placements for a {ndim}-D mesh: the "
                             "convention [Shard(1), Shard(2), ...] would shard the FEATURE axis. Pass placements= "
                             "explicitly (e.g. [Replicate(), Shard(1), Shard(2)] for a dp x cp x cp mesh).")
        from torch.distributed.tensor import Shard

        return [Shard(tensor_dim) for tensor_dim in range(1, ndim + 1)]

    def _resolve_cp(self, device_mesh, placements):
        """``(cp, cp_axis_sizes, pe_map)``; ``(1, (), None)`` when nothing is split.  Touches no
        symmetric memory: a module can be constructed before ``init_nvshmem()``."""
        nothing_split = (1, (), None)
        if device_mesh is None or placements is None or int(device_mesh.mesh.numel()) == 1:
            return nothing_split
        if _token_split_factor(device_mesh, _effective_placements(device_mesh, placements)) <= 1:
            return nothing_split
        validate_trimul_sharding(placements, device_mesh.ndim)
        pe_map = PeMap.from_mesh_placements(device_mesh, _token_placements(device_mesh, placements),
                                            distributed_manager=self._dm)
        return int(pe_map.cp), tuple(int(s) for s in pe_map.cp_axis_sizes), pe_map

    # -- introspection -------------------------------------------------------------------------
    @property
    def incoming_variant(self) -> str:
        """``"cp1_fallback"`` (single-GPU routing), ``"unbuilt"``, one of
        :data:`INCOMING_STORE_VARIANTS`, or ``"mixed"``."""
        if self._cp == 1:
            return "cp1_fallback"
        built = sorted(set(self._engine_variant.values()))
        if not built:
            return "unbuilt"
        return built[0] if len(built) == 1 else "mixed"

    def check(self) -> None:
        """Synchronise and raise :class:`fold_cp_ops_b200.kernels.DeviceWaitTimeout` (a
        ``CollectiveError``) if a bounded device-side wait of any forward issued so far expired --
        outputs of that forward are invalid.  The next ``forward`` makes the same check without
        synchronising.  A cp=1 module checks the single-GPU engine that served it."""
        for eng in self._live_engines():
            eng.check()

    def last_forward_stats(self) -> dict:
        """Statistics of the last forward run with ``collect_stats(True)``: per-kernel ms, ms spent in
        each cross-rank flag wait (all-to-all time not hidden behind a kernel), device-clock spans and
        bytes stored into peers' buffers.  Empty before the first such forward."""
        for eng in self._live_engines():
            stats = eng.last_forward_stats()
            if stats:
                return stats
        return {}

    def collect_stats(self, enabled: bool = True) -> None:
        """Switch the per-forward measurements on or off (they cost six event records and one 128-byte
        copy per forward)."""
        self._collect_stats = bool(enabled)
        for eng in self._live_engines():
            eng.collect_stats = self._collect_stats

    def _live_engines(self):
        if self._cp > 1:
            return list(self._engines.values())
        from ...workflows import trimul_autotune as single

        return single.engines_for_weights(self._w)

    # -- the three public verbs ----------------------------------------------------------------
    def prepare(self, *, n_token: int, batch: int = 1, masked: bool = False):
        """Build the ``(batch, masked)`` engine and allocate its symmetric buffers for ``n_token``.
        Optional and idempotent; ``forward`` calls it for whatever arrives.  Returns the engine, or
        ``None`` for a cp == 1 module.  COLLECTIVE for cp > 1."""
        if int(n_token) < 1 or int(batch) < 1:
            raise ValueError(f"n_token and batch must be >= 1; got {n_token!r}, {batch!r}")
        if self._cp == 1:
            return None
        key = (int(batch), bool(masked))
        if key not in self._engines:
            kw = _store_variant_kwargs(dict(self._kw), self._dir, self._cp1, int(batch))
            _ensure_nvshmem(self._dm)
            eng = TriMulAutotuned(self._pe_map, int(batch), int(n_token), self._D, self._w, self._dt,
                                  device_mesh=self.device_mesh, placements=self._placements, dynamic=True,
                                  has_mask=bool(masked), eps=self._eps, **kw)
            eng.collect_stats = getattr(self, "_collect_stats", False)
            self._engines[key] = eng
            self._engine_variant[key] = eng.store_variant
        return self._engines[key]

    def _refuse_foreign_input(self, x) -> None:
        """The three ways an input can disagree with what the module was built for."""
        x_mesh = getattr(x, "device_mesh", None)
        if x_mesh is not None and self.device_mesh is not None and x_mesh is not self.device_mesh \
                and x_mesh != self.device_mesh:
            raise ValueError(f"TriangularMultiplication was constructed on device_mesh={self.device_mesh}, but "
                             f"forward() received a DTensor on {x_mesh}. The cached fused instance is built for "
                             "the constructor's mesh; running it against another one would reshard onto a peer "
                             "map it was not built for.")
        if self._cp == 1 or _is_single_device(x):
            return
        given = list(_dtensor_mesh_placements(x)[1])
        if given != list(self._placements):
            raise ValueError(f"TriangularMultiplication was built for placements={self._placements}, but forward() "
                             f"received a DTensor placed {given}. The PeMap and the peer stores are derived "
                             "from the constructor's placements; running against another sharding would all-to-all "
                             "over a different set of peers. Pass placements= to the constructor if this module's "
                             "sharding is not the default [Shard(i + 1) for i in range(mesh.ndim)].")
        if int(x.shape[3]) != self._D:
            raise ValueError(f"TriangularMultiplication holds weights of feature width D={self._D} (from norm_in), "
                             f"but forward() received a tensor of width {int(x.shape[3])}. The projections would "
                             "not contract.")

    @torch.no_grad()
    def forward(self, x, mask=None):
        """DTensor ``(B, N, N, D)`` -> DTensor of the same sharding (plain tensor -> plain tensor)."""
        self._refuse_foreign_input(x)
        if self._cp == 1 or _is_single_device(x):
            return _trimul_single_device(x, self._w, direction=self._dir, mask=mask, eps=self._eps)
        key = (int(x.shape[0]), mask is not None)
        if key not in self._engines:
            self._warn_second_variant(key)
        eng = self.prepare(n_token=int(x.shape[1]), batch=key[0], masked=key[1])
        return _rewrap_like(x, eng.forward(_local(x), self._dir, mask_local=_local(mask)))

    def _warn_second_variant(self, key) -> None:
        """A second ``(batch, masked)`` engine doubles the symmetric memory the module holds: say so, once."""
        if self._engines and not self._warned_second_variant:
            self._warned_second_variant = True
            warnings.warn(f"TriangularMultiplication is building a SECOND engine: it already holds (batch, masked)="
                          f"{sorted(self._engines)} and forward() was called with {key}. Each engine holds its own set "
                          "of symmetric receive buffers for the module's lifetime. If the batch extent genuinely varies "
                          "per call this is expected; if it does not, the shapes disagree. Warned once.",
                          RuntimeWarning, stacklevel=3)

    def free(self):
        """Drop every engine's buffers.  No collective runs here (symmetric blocks return to their
        pool by refcount), so ranks may call it in any order; a no-op for a cp=1 module."""
        while self._engines:
            _, eng = self._engines.popitem()
            try:
                eng.free()
            except Exception as exc:  # noqa: BLE001 - teardown must not raise
                warnings.warn(f"engine free() raised (ignored): {exc!r}")
        self._engine_variant.clear()
