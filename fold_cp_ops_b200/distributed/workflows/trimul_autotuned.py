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
"""
from __future__ import annotations

import difflib
import inspect
import warnings
from typing import Optional

import numpy as np
import torch
import torch.nn as nn

from ...engine import CpGeometry, TriMulEngine
from ...workflows.trimul_autotune import trimul_autotuned
from ..dtensor_adapter import (_dtensor_mesh_placements, _effective_placements, _ensure_nvshmem, _is_dtensor,
                               _rowmaj_stride, _token_split_factor, validate_trimul_sharding)
from ..pe_map import PeMap, _is_shard, _mesh_rank_tensor, _placement_shard_dim
from ..trimul_weights import W_KEYS, W_PROJ_BIAS_KEYS
from .trimul_tuning import IGNORED_ON_SM100, TriMulTuning

__all__ = ["TriangularMultiplication", "trimul_a2a"]

_W_ALL_KEYS = tuple(W_KEYS) + tuple(W_PROJ_BIAS_KEYS)
_TRIMUL_NON_W = ("x", "mask", "direction", "eps", "out", "select", "_config")
_TRIMUL_W_KWARGS = tuple(p for p in inspect.signature(trimul_autotuned).parameters if p not in _TRIMUL_NON_W)
assert set(_W_ALL_KEYS) == set(_TRIMUL_W_KWARGS), (
    "trimul_weights.W_KEYS + W_PROJ_BIAS_KEYS must be EXACTLY trimul_autotuned's weight kwargs; only in w: "
    f"{sorted(set(_W_ALL_KEYS) - set(_TRIMUL_W_KWARGS))}; only in trimul_autotuned: "
    f"{sorted(set(_TRIMUL_W_KWARGS) - set(_W_ALL_KEYS))}")
_W_LN_KEYS = ("norm_in_w", "norm_in_b", "norm_out_w", "norm_out_b")

#: front-store variants of the incoming path.  They name RECEIVE LAYOUTS of the reference; this
#: build always writes the transposed operand plane for "incoming", and reports the reference's
#: name for the configuration so callers that record it keep working.
INCOMING_STORE_VARIANTS = ("plain", "composite_k", "route2_ni")


# ---------------------------------------------------------------------------------------------
# cp=1 routing and re-wrapping
# ---------------------------------------------------------------------------------------------
def _is_single_device(x) -> bool:
    """True when nothing needs communicating: a plain tensor, a one-device mesh, or placements
    that split neither token axis (this includes a dp-only mesh with ``Shard(0)``)."""
    if not _is_dtensor(x):
        return True
    mesh, placements = _dtensor_mesh_placements(x)
    if mesh is None or int(mesh.mesh.numel()) == 1:
        return True
    return _token_split_factor(mesh, _effective_placements(mesh, placements)) <= 1


def _rewrap_like(x, out_local):
    """Plain in -> plain out; DTensor in -> DTensor with ``x``'s mesh, placements and global shape."""
    if not _is_dtensor(x):
        return out_local
    from torch.distributed.tensor import DTensor

    mesh, placements = _dtensor_mesh_placements(x)
    shape = tuple(x.shape)
    return DTensor.from_local(out_local, mesh, list(placements), shape=torch.Size(shape),
                              stride=_rowmaj_stride(shape), run_check=False)


def _trimul_single_device(x, w: dict, *, direction: str, mask, eps: float = 1e-5):
    unexpected = [k for k in w if k not in _W_ALL_KEYS]
    if unexpected:
        raise KeyError(f"cp=1 TriMul fallback got unexpected weight key(s) {sorted(unexpected)}; "
                       f"expected exactly {list(_W_ALL_KEYS)}")
    wk = {k: w.get(k) for k in _W_ALL_KEYS}
    for k in _W_LN_KEYS:
        if wk[k] is not None:
            wk[k] = wk[k].float()
    x_local = x.to_local() if _is_dtensor(x) else x
    mask_local = mask.to_local() if _is_dtensor(mask) else mask
    out_local = trimul_autotuned(x_local, **wk, mask=mask_local, direction=direction, eps=eps, select="heuristic")
    return _rewrap_like(x, out_local)


def incoming_store_variant(direction: str, cp1: int, batch: int = 1) -> str:
    """``plain`` | ``composite_k`` | ``route2_ni`` as a total function of ``(direction, cp1)``:
    outgoing -> plain; incoming on a 1-D token shard -> composite_k; incoming on 2-D -> route2_ni.
    ``batch`` is validated (>= 1) and otherwise ignored."""
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}. Falling through to "
                         "the plain store on a typo would silently cost ~2x on the incoming path.")
    if int(cp1) < 1:
        raise ValueError(f"cp1 must be >= 1; got {cp1!r}")
    if int(batch) < 1:
        raise ValueError(f"batch must be >= 1; got {batch!r}")
    if direction == "outgoing":
        return "plain"
    return "composite_k" if int(cp1) == 1 else "route2_ni"


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
    (always dynamic).  Keywords that configured SM90 tiles or NVSHMEM drains are accepted and
    ignored (``trimul_tuning.IGNORED_ON_SM100``)."""

    def __init__(self, pe_map: PeMap, B: int, N: int, D: int, w: dict, dt: torch.dtype, *, device_mesh=None,
                 placements=None, dynamic: bool = True, has_mask: bool = False, eps: float = 1e-5,
                 composite_k: bool = False, route2_ni: bool = False, front_tile_mn=None, front_pad_inner=None,
                 front_pad_eager=None, back_tile_mn=None, back_pingpong=None, back_cluster_n=None, consumer=None,
                 use_device_signal_nvlink=None, autotune_config=None, is_persistent=None, allocate: bool = True):
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
        super().__init__(w, device=pe_map.device, eps=eps, geometry=geometry, process_group=group)
        self.pe_map = pe_map
        self.has_mask = bool(has_mask)
        self.composite_k = bool(composite_k)
        self.route2_ni = bool(route2_ni)
        self.dynamic = True
        if allocate:
            self.prepare(int(B), int(N))

    def forward(self, x_local, direction, mask_local=None):  # noqa: D102 - documented on the base class
        return super().forward(x_local, direction, mask_local)


def _reject_unknown_engine_kwargs(fused_kwargs: dict) -> None:
    """Refuse, at the call the user wrote, a keyword the engine constructor does not have."""
    legal = {n for n, prm in inspect.signature(TriMulAutotuned.__init__).parameters.items()
             if prm.kind is inspect.Parameter.KEYWORD_ONLY}
    unknown = sorted(set(fused_kwargs) - legal)
    if not unknown:
        return
    hints = []
    for k in unknown:
        near = difflib.get_close_matches(k, sorted(legal), n=1)
        hints.append(f"{k!r}" + (f" (did you mean {near[0]!r}?)" if near else ""))
    raise TypeError(f"trimul_a2a got unknown fused_kwargs: {', '.join(hints)}. Legal engine knobs are {sorted(legal)}. "
                    "Refused here rather than inside the lazy engine build, which happens after the PeMap and the "
                    "symmetric buffers are up and reports a TypeError from a constructor you did not call.")


def _build_pe_map(x, distributed_manager):
    mesh, placements = _dtensor_mesh_placements(x)
    validate_trimul_sharding(placements, mesh.ndim)
    pe_map = PeMap.from_mesh_placements(mesh, _token_placements(mesh, placements),
                                        distributed_manager=distributed_manager)
    return pe_map, mesh, placements


def _get_engine(cache, pe_map, mesh, placements, B, N, D, w, dt, *, dynamic, has_mask, kw):
    key = (B, None if dynamic else int(N), int(D), pe_map.cp, tuple(int(s) for s in pe_map.cp_axis_sizes),
           bool(has_mask), bool(kw.get("composite_k", False)), bool(kw.get("route2_ni", False)))
    inst = cache.get(key)
    if inst is None:
        _ensure_nvshmem(kw.get("distributed_manager"))
        ctor_kw = {k: v for k, v in kw.items() if k != "distributed_manager"}
        inst = TriMulAutotuned(pe_map, B, int(N), int(D), w, dt, device_mesh=mesh, placements=placements,
                               dynamic=dynamic, has_mask=has_mask, **ctor_kw)
        cache[key] = inst
    return inst


_FUSED_CACHE: dict = {}


def trimul_a2a(x, w: dict, dt: torch.dtype, *, direction: str = "outgoing", mask=None, dynamic: bool = True,
               distributed_manager=None, _cache: Optional[dict] = None, **fused_kwargs):
    """Functional form: DTensor ``(B, N, N, D)`` -> same-sharding DTensor.  Inference only.

    ``w`` is the replicated 12-key weight dict; ``mask`` a DTensor sharded like ``x``, a local
    tensor or ``None``.  cp == 1 inputs short-circuit to the single-GPU ``trimul_autotuned`` before
    any peer map is built.  ``_cache`` lets a caller own the engine cache; ``None`` uses a
    process-global one."""
    assert direction in ("outgoing", "incoming"), "direction must be 'outgoing'|'incoming'"
    _reject_unknown_engine_kwargs(fused_kwargs)
    if not _is_dtensor(x) and not isinstance(x, torch.Tensor):
        raise TypeError(f"trimul_a2a expects a DTensor or local Tensor x, got {type(x)}.")
    if _is_single_device(x):
        return _trimul_single_device(x, w, direction=direction, mask=mask, eps=fused_kwargs.get("eps", 1e-5))
    cache = _FUSED_CACHE if _cache is None else _cache
    pe_map, mesh, placements = _build_pe_map(x, distributed_manager)
    B, N, _, D = x.shape
    kw = dict(fused_kwargs)
    kw["distributed_manager"] = distributed_manager
    cp_axis = tuple(int(s) for s in pe_map.cp_axis_sizes)
    cp1 = cp_axis[1] if len(cp_axis) > 1 else 1
    if "composite_k" not in kw and "route2_ni" not in kw:
        variant = incoming_store_variant(direction, cp1, int(B))
        if variant != "plain":
            kw[variant] = True
    eng = _get_engine(cache, pe_map, mesh, placements, int(B), int(N), int(D), w, dt, dynamic=dynamic,
                      has_mask=mask is not None, kw=kw)
    mask_local = mask.to_local() if _is_dtensor(mask) else mask
    out_local = eng.forward(x.to_local(), direction, mask_local=mask_local)
    return _rewrap_like(x, out_local)


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

    def __init__(self, layer: nn.Module, direction: str, device_mesh, distributed_manager, *, placements=None,
                 dtype: torch.dtype = torch.bfloat16, eps: Optional[float] = None,
                 tuning: Optional[TriMulTuning] = None):
        super().__init__()
        if direction not in ("outgoing", "incoming"):
            raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}. It selects the "
                             "back-half einsum, so an unrecognised value would compute a different contraction.")
        from ..trimul_weights import weights_from_trimul_module

        w = weights_from_trimul_module(layer)
        for k in _W_LN_KEYS:
            if w[k] is not None and w[k].dtype is not torch.float32:
                w[k] = w[k].float()
        self._w = w
        self._dt = dtype
        self._dir = direction
        self._dm = distributed_manager
        if eps is None:
            eps = float(getattr(getattr(layer, "norm_in", None), "eps", 1e-5))
        self._eps = float(eps)
        self._tuning = tuning
        self._kw = tuning.to_engine_kwargs() if tuning is not None else {}
        self.device_mesh = device_mesh
        self.direction = direction
        self._D = int(w["norm_in_w"].shape[0])
        self._placements = self._resolve_placements(device_mesh, placements)
        self._cp, self._cp_axis_sizes, self._pe_map = self._resolve_cp(device_mesh, self._placements)
        self._cp1 = int(self._cp_axis_sizes[1]) if len(self._cp_axis_sizes) > 1 else 1
        self._engines: dict = {}
        self._engine_variant: dict = {}
        self._warned_second_variant = False
        self.norm_in = layer.norm_in
        self.p_in = layer.p_in
        self.g_in = layer.g_in
        self.norm_out = layer.norm_out
        self.p_out = layer.p_out
        self.g_out = layer.g_out

    @staticmethod
    def _resolve_placements(device_mesh, placements):
        if device_mesh is None:
            return None if placements is None else list(placements)
        if not hasattr(device_mesh, "ndim") or not hasattr(device_mesh, "mesh"):
            raise TypeError(f"device_mesh must be a DeviceMesh (it needs .ndim and .mesh) or None; got "
                            f"{type(device_mesh).__name__}. The constructor derives cp, the placements and the "
                            "PeMap from it, so an object that only compares equal is not enough.")
        ndim = int(device_mesh.ndim)
        if placements is not None:
            pl = list(placements)
            if len(pl) != ndim:
                raise ValueError(f"placements has {len(pl)} entries but device_mesh.ndim is {ndim}. One placement "
                                 "per mesh dim is required; there is no padding rule.")
            return pl
        if ndim > 2:
            raise ValueError(f"TriangularMultiplication cannot default the placements for a {ndim}-D mesh: the "
                             "convention [Shard(1), Shard(2), ...] would shard the FEATURE axis. Pass placements= "
                             "explicitly (e.g. [Replicate(), Shard(1), Shard(2)] for a dp x cp x cp mesh).")
        from torch.distributed.tensor import Shard

        return [Shard(i + 1) for i in range(ndim)]

    def _resolve_cp(self, device_mesh, placements):
        """``(cp, cp_axis_sizes, pe_map)``; ``(1, (), None)`` when nothing is split.  Touches no
        symmetric memory: a module can be constructed before ``init_nvshmem()``."""
        if device_mesh is None or placements is None or int(device_mesh.mesh.numel()) == 1:
            return 1, (), None
        eff = _effective_placements(device_mesh, placements)
        if _token_split_factor(device_mesh, eff) <= 1:
            return 1, (), None
        validate_trimul_sharding(placements, device_mesh.ndim)
        pe_map = PeMap.from_mesh_placements(device_mesh, _token_placements(device_mesh, placements),
                                            distributed_manager=self._dm)
        return int(pe_map.cp), tuple(int(s) for s in pe_map.cp_axis_sizes), pe_map

    @property
    def incoming_variant(self) -> str:
        """``"cp1_fallback"`` (single-GPU routing), ``"unbuilt"``, one of
        :data:`INCOMING_STORE_VARIANTS`, or ``"mixed"``."""
        if self._cp == 1:
            return "cp1_fallback"
        vs = set(self._engine_variant.values())
        if not vs:
            return "unbuilt"
        return vs.pop() if len(vs) == 1 else "mixed"

    def prepare(self, *, n_token: int, batch: int = 1, masked: bool = False):
        """Build the ``(batch, masked)`` engine and allocate its symmetric buffers for ``n_token``.
        Optional and idempotent; ``forward`` calls it for whatever arrives.  Returns the engine, or
        ``None`` for a cp == 1 module.  COLLECTIVE for cp > 1."""
        if int(n_token) < 1 or int(batch) < 1:
            raise ValueError(f"n_token and batch must be >= 1; got {n_token!r}, {batch!r}")
        if self._cp == 1:
            return None
        key = (int(batch), bool(masked))
        eng = self._engines.get(key)
        if eng is not None:
            return eng
        variant = incoming_store_variant(self._dir, self._cp1, int(batch))
        kw = dict(self._kw)
        if variant != "plain" and "composite_k" not in kw and "route2_ni" not in kw:
            kw[variant] = True
        _ensure_nvshmem(self._dm)
        eng = TriMulAutotuned(self._pe_map, int(batch), int(n_token), self._D, self._w, self._dt,
                              device_mesh=self.device_mesh, placements=self._placements, dynamic=True,
                              has_mask=bool(masked), eps=self._eps, **kw)
        self._engines[key] = eng
        self._engine_variant[key] = "composite_k" if eng.composite_k else ("route2_ni" if eng.route2_ni else "plain")
        return eng

    @torch.no_grad()
    def forward(self, x, mask=None):
        """DTensor ``(B, N, N, D)`` -> DTensor of the same sharding (plain tensor -> plain tensor)."""
        x_mesh = getattr(x, "device_mesh", None)
        if x_mesh is not None and self.device_mesh is not None and x_mesh is not self.device_mesh:
            if x_mesh != self.device_mesh:
                raise ValueError(f"TriangularMultiplication was constructed on device_mesh={self.device_mesh}, but "
                                 f"forward() received a DTensor on {x_mesh}. The cached fused instance is built for "
                                 "the constructor's mesh; running it against another one would reshard onto a peer "
                                 "map it was not built for.")
        if self._cp == 1 or _is_single_device(x):
            return _trimul_single_device(x, self._w, direction=self._dir, mask=mask, eps=self._eps)
        _, x_pl = _dtensor_mesh_placements(x)
        if list(x_pl) != list(self._placements):
            raise ValueError(f"TriangularMultiplication was built for placements={self._placements}, but forward() "
                             f"received a DTensor placed {list(x_pl)}. The PeMap and the peer stores are derived "
                             "from the constructor's placements; running against another sharding would all-to-all "
                             "over a different set of peers. Pass placements= to the constructor if this module's "
                             "sharding is not the default [Shard(i + 1) for i in range(mesh.ndim)].")
        if int(x.shape[3]) != self._D:
            raise ValueError(f"TriangularMultiplication holds weights of feature width D={self._D} (from norm_in), "
                             f"but forward() received a tensor of width {int(x.shape[3])}. The projections would "
                             "not contract.")
        key = (int(x.shape[0]), mask is not None)
        eng = self._engines.get(key)
        if eng is None:
            self._warn_second_variant(key)
            eng = self.prepare(n_token=int(x.shape[1]), batch=key[0], masked=key[1])
        mask_local = mask.to_local() if _is_dtensor(mask) else mask
        out_local = eng.forward(x.to_local(), self._dir, mask_local=mask_local)
        return _rewrap_like(x, out_local)

    def _warn_second_variant(self, key) -> None:
        if self._warned_second_variant or not self._engines:
            return
        self._warned_second_variant = True
        warnings.warn(f"TriangularMultiplication is building a SECOND engine: it already holds (batch, masked)="
                      f"{sorted(self._engines)} and forward() was called with {key}. Each engine holds its own set "
                      "of symmetric receive buffers for the module's lifetime. If the batch extent genuinely varies "
                      "per call this is expected; if it does not, the shapes disagree. Warned once.",
                      RuntimeWarning, stacklevel=3)

    def free(self):
        """Drop every engine's buffers.  No collective runs here (symmetric blocks return to their
        pool by refcount), so ranks may call it in any order; a no-op for a cp=1 module."""
        for inst in self._engines.values():
            try:
                inst.free()
            except Exception as exc:  # noqa: BLE001 - teardown must not raise
                warnings.warn(f"engine free() raised (ignored): {exc!r}")
        self._engines.clear()
        self._engine_variant.clear()
