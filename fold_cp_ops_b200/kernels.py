"""Per-kernel Python entry points over the C ABI, taking torch CUDA tensors.

Each function checks dtypes / contiguity, passes raw device pointers and the current CUDA stream
to ``libtrimul_sm100.so`` and returns nothing: outputs are written into caller-provided tensors.
They are the unit the parity tests and the profiler drive; the engine chains them.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from .distributed.collective_symmetry import CollectiveError

DEFAULT_TIMEOUT_NS = 2_000_000_000

_MASK_KINDS = {torch.bfloat16: _lib.MASK_BF16, torch.float32: _lib.MASK_FP32,
               torch.uint8: _lib.MASK_U8, torch.bool: _lib.MASK_U8}


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor; the TriMul kernels have no CPU path")
    if t.dtype is not dtype:
        raise ValueError(f"{name} must be {dtype}; got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def make_geom(batch: int, n: int, d: int, direction: str, eps: float, cp0: int = 1, cp1: int = 1,
              rank: int = 0) -> _lib.Geom:
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}")
    return _lib.Geom(int(batch), int(n), int(d), int(cp0), int(cp1), int(rank),
                     _lib.OUTGOING if direction == "outgoing" else _lib.INCOMING, float(eps))


def device_caps(device: int) -> _lib.Caps:
    """Query the device and raise unless it is compute capability 10.x."""
    caps = _lib.Caps()
    rc = _lib.load().trimul_sm100_query(int(device), C.byref(caps))
    if rc == _lib.ERR_UNSUPPORTED_ARCH:
        raise RuntimeError(_lib.last_error())
    _lib.check(rc, "trimul_sm100_query")
    return caps


def workspace_bytes(geom: _lib.Geom) -> _lib.Workspace:
    ws = _lib.Workspace()
    _lib.check(_lib.load().trimul_sm100_workspace(C.byref(geom), C.byref(ws)), "trimul_sm100_workspace")
    return ws


def reshard_plan(geom: _lib.Geom) -> _lib.ReshardPlan:
    """Host-side index arithmetic of the two fused reshards for this rank (no device work)."""
    plan = _lib.ReshardPlan()
    _lib.check(_lib.load().trimul_sm100_reshard_plan(C.byref(geom), C.byref(plan)), "trimul_sm100_reshard_plan")
    return plan


def contract_walk(geom: _lib.Geom, tuning: Optional[_lib.Tuning] = None):
    """``((tiles_i, tiles_j), [(tile_row, tile_col), ...])``: the order in which the contraction kernel visits
    the tiles of one channel plane for this rank and tuning (host-side; no device work)."""
    lib = _lib.load()
    ti, tj = C.c_int32(0), C.c_int32(0)
    ref = None if tuning is None else C.byref(tuning)
    _lib.check(lib.trimul_sm100_contract_walk(C.byref(geom), ref, 0, None, None, C.byref(ti), C.byref(tj)),
               "trimul_sm100_contract_walk")
    n = ti.value * tj.value
    rows, cols = (C.c_int32 * n)(), (C.c_int32 * n)()
    _lib.check(lib.trimul_sm100_contract_walk(C.byref(geom), ref, n, rows, cols, C.byref(ti), C.byref(tj)),
               "trimul_sm100_contract_walk")
    return (ti.value, tj.value), list(zip(rows, cols))


def new_status(device) -> torch.Tensor:
    """A zeroed device status record (8 x int32) for the bounded waits to report into."""
    return torch.zeros(8, dtype=torch.int32, device=device)


class DeviceWaitTimeout(CollectiveError):
    """A bounded device-side wait expired; the kernel returned early and the CUDA context is intact.

    A member of the ``CollectiveError`` family: the usual cause is a peer rank that never delivered
    its half of a reshard, and the right reaction is the same -- do not enter another collective
    with outputs of this forward."""


_KERNEL_NAMES = {1: "ln_gated_proj", 2: "tri_contract", 3: "ln_out_proj", 4: "peer_sync"}


def describe_status(record: Sequence[int]) -> str:
    """The sentence a status record (8 x int32 as a list) stands for."""
    if record[1] == 4:
        slot = {0: "FRONT", 1: "BACK", 2: "CONSUMED"}.get(record[3], str(record[3]))
        return (f"a cross-rank flag wait expired: counter {slot} stood at {record[4]} when the bound ran out -- a "
                "peer rank did not deliver its half of a reshard; outputs of this forward are invalid")
    return (f"bounded wait expired in kernel {_KERNEL_NAMES.get(record[1], record[1])}: block {record[2]}, role "
            f"{record[3]}, detail {record[4]}; outputs of this forward are invalid")


def check_status(status: torch.Tensor) -> None:
    """Synchronising read of the status record; raises :class:`DeviceWaitTimeout` if a wait expired."""
    s = status.tolist()
    if s[0] != 0:
        status.zero_()
        raise DeviceWaitTimeout(describe_status(s))


def pack_weights(d: int, p_in_w, g_in_w, g_out_w, p_in_b=None, g_in_b=None, g_out_b=None):
    """Regroup the input-side weights into the chunk order the projection kernel streams.

    Returns ``(w_packed (5d, d) bf16, bias_packed (5d,) fp32)``.
    """
    for t, nm, shp in ((p_in_w, "p_in_w", (2 * d, d)), (g_in_w, "g_in_w", (2 * d, d)), (g_out_w, "g_out_w", (d, d))):
        _require(t, torch.bfloat16, nm)
        if tuple(t.shape) != shp:
            raise ValueError(f"{nm} must have shape {shp}; got {tuple(t.shape)}")
    for t, nm in ((p_in_b, "p_in_b"), (g_in_b, "g_in_b"), (g_out_b, "g_out_b")):
        if t is not None:
            _require(t, torch.float32, nm)
    dev = p_in_w.device
    w_packed = torch.empty(5 * d, d, dtype=torch.bfloat16, device=dev)
    bias_packed = torch.empty(5 * d, dtype=torch.float32, device=dev)
    rc = _lib.load().trimul_sm100_pack_weights(d, _ptr(p_in_w), _ptr(g_in_w), _ptr(g_out_w), _ptr(p_in_b),
                                               _ptr(g_in_b), _ptr(g_out_b), _ptr(w_packed), _ptr(bias_packed),
                                               _stream())
    _lib.check(rc, "trimul_sm100_pack_weights")
    return w_packed, bias_packed


def _mask_args(mask: Optional[torch.Tensor]):
    if mask is None:
        return None, _lib.MASK_NONE
    if not mask.is_cuda or not mask.is_contiguous():
        raise ValueError("mask must be a contiguous CUDA tensor")
    kind = _MASK_KINDS.get(mask.dtype)
    if kind is None:
        raise ValueError(f"mask dtype {mask.dtype} is not supported (bf16, fp32, uint8, bool)")
    return mask.data_ptr(), kind


def _ptr_array(ptrs: Sequence[int]):
    arr = (C.c_void_p * len(ptrs))(*[C.c_void_p(int(p)) for p in ptrs])
    return arr


def make_tuning(contract_form: str = "auto", front_fixed_order: bool = False, contract_band_rows: int = 0,
                contract_fixed_start: bool = False, contract_pace_ns: int = 0) -> _lib.Tuning:
    """The library's tuning record: ``contract_form`` is ``"auto"`` (CTA pairs whenever the device has two
    SMs), ``"single"`` (one CTA per 128 x 256 tile) or ``"pair"`` (two CTAs per 256 x 256 tile);
    ``contract_band_rows`` is the height, in tile rows, of the bands the contraction walks column by
    column (0: the library's choice, 1: row-major); ``contract_fixed_start`` makes every rank walk from
    tile (0, 0) instead of from its own block of the result; ``contract_pace_ns`` (<= 100000; 0 = the
    library's choice, negative = off) is the longest a CTA pair waits before a tile for the other pairs to
    start theirs (a hint that keeps tiles sharing operand strips in step; results never depend on it)."""
    if int(contract_pace_ns) > 100000:
        raise ValueError(f"contract_pace_ns must be <= 100000; got {contract_pace_ns}")
    if int(contract_band_rows) < 0:
        raise ValueError(f"contract_band_rows must be >= 0; got {contract_band_rows}")
    forms = {"auto": _lib.CONTRACT_DEFAULT, "single": _lib.CONTRACT_SINGLE, "pair": _lib.CONTRACT_PAIR}
    if contract_form not in forms:
        raise ValueError(f"contract_form must be one of {sorted(forms)}; got {contract_form!r}")
    t = _lib.Tuning()
    t.contract_form = forms[contract_form]
    t.front_fixed_order = 1 if front_fixed_order else 0
    t.contract_band_rows = int(contract_band_rows)
    t.contract_fixed_start = 1 if contract_fixed_start else 0
    t.contract_pace_ns = int(contract_pace_ns)
    return t


def _tuning_ref(tuning):
    return None if tuning is None else C.byref(tuning)


def ln_gated_proj(geom, x, mask, ln_w, ln_b, w_packed, bias_packed, ab_peer_ptrs: Sequence[int], gate_out,
                  status, timeout_ns: int = DEFAULT_TIMEOUT_NS, tuning=None) -> None:
    _require(x, torch.bfloat16, "x")
    _require(ln_w, torch.float32, "ln_w")
    if ln_b is not None:
        _require(ln_b, torch.float32, "ln_b")
    _require(gate_out, torch.bfloat16, "gate_out")
    mptr, mkind = _mask_args(mask)
    rc = _lib.load().trimul_sm100_ln_gated_proj(C.byref(geom), _tuning_ref(tuning), _ptr(x), mptr, mkind, _ptr(ln_w), _ptr(ln_b),
                                                _ptr(w_packed), _ptr(bias_packed), _ptr_array(ab_peer_ptrs),
                                                _ptr(gate_out), _ptr(status), int(timeout_ns), _stream())
    _lib.check(rc, "trimul_sm100_ln_gated_proj")


def tri_contract(geom, ab_local, tri_peer_ptrs: Sequence[int], status, timeout_ns: int = DEFAULT_TIMEOUT_NS,
                 tuning=None) -> None:
    _require(ab_local, torch.bfloat16, "ab_local")
    rc = _lib.load().trimul_sm100_tri_contract(C.byref(geom), _tuning_ref(tuning), _ptr(ab_local), _ptr_array(tri_peer_ptrs),
                                               _ptr(status), int(timeout_ns), _stream())
    _lib.check(rc, "trimul_sm100_tri_contract")


def pack_out_weights(d: int, p_out_w, ln_w, ln_b=None, p_out_b=None):
    """Fold the output LayerNorm into the output projection.

    Returns ``(w_fold (d, d) bf16 = bf16(ln_w * W), cd (d, 2) fp32 = (sum_k w_fold, sum_k ln_b*W + bias))``.
    """
    _require(p_out_w, torch.bfloat16, "p_out_w")
    _require(ln_w, torch.float32, "ln_w")
    if tuple(p_out_w.shape) != (d, d):
        raise ValueError(f"p_out_w must have shape {(d, d)}; got {tuple(p_out_w.shape)}")
    for t, nm in ((ln_b, "ln_b"), (p_out_b, "p_out_b")):
        if t is not None:
            _require(t, torch.float32, nm)
    w_fold = torch.empty(d, d, dtype=torch.bfloat16, device=p_out_w.device)
    cd = torch.empty(d, 2, dtype=torch.float32, device=p_out_w.device)
    rc = _lib.load().trimul_sm100_pack_out_weights(d, _ptr(p_out_w), _ptr(ln_w), _ptr(ln_b), _ptr(p_out_b),
                                                   _ptr(w_fold), _ptr(cd), _stream())
    _lib.check(rc, "trimul_sm100_pack_out_weights")
    return w_fold, cd


def ln_out_proj(geom, tri_local, gate, w_fold, cd, out, status, timeout_ns: int = DEFAULT_TIMEOUT_NS) -> None:
    _require(tri_local, torch.bfloat16, "tri_local")
    _require(gate, torch.bfloat16, "gate")
    _require(w_fold, torch.bfloat16, "w_fold")
    _require(cd, torch.float32, "cd")
    _require(out, torch.bfloat16, "out")
    rc = _lib.load().trimul_sm100_ln_out_proj(C.byref(geom), _ptr(tri_local), _ptr(gate), _ptr(w_fold), _ptr(cd),
                                              _ptr(out), _ptr(status), int(timeout_ns), _stream())
    _lib.check(rc, "trimul_sm100_ln_out_proj")


def forward_single(geom, x, mask, ln_in_w, ln_in_b, w_packed, bias_packed, w_fold, cd, ab, tri, gate, out, status,
                   timeout_ns: int = DEFAULT_TIMEOUT_NS) -> None:
    """The whole cp=1 chain through ``trimul_sm100_forward``."""
    _require(x, torch.bfloat16, "x")
    _require(out, torch.bfloat16, "out")
    mptr, mkind = _mask_args(mask)
    rc = _lib.load().trimul_sm100_forward(C.byref(geom), _ptr(x), mptr, mkind, _ptr(ln_in_w), _ptr(ln_in_b),
                                          _ptr(w_packed), _ptr(bias_packed), _ptr(w_fold), _ptr(cd), _ptr(ab),
                                          _ptr(tri), _ptr(gate), _ptr(out), _ptr(status), int(timeout_ns), _stream())
    _lib.check(rc, "trimul_sm100_forward")


def forward_static(geom, x, mask, ln_in_w, ln_in_b, w_packed, bias_packed, w_fold, cd, out, status,
                   timeout_ns: int = DEFAULT_TIMEOUT_NS) -> None:
    """The cp=1 chain with the library's built-in scratch array instead of caller buffers.

    For callers that cannot allocate device memory: no tensor is created here and the library
    allocates nothing.  Shapes need ``8 * batch * n * n * d <= STATIC_SCRATCH_BYTES`` (32 MiB);
    larger ones raise ``ValueError``.  Calls that overlap on the GPU share the one array and race.
    """
    _require(x, torch.bfloat16, "x")
    _require(out, torch.bfloat16, "out")
    mptr, mkind = _mask_args(mask)
    rc = _lib.load().trimul_sm100_forward_static(C.byref(geom), _ptr(x), mptr, mkind, _ptr(ln_in_w), _ptr(ln_in_b),
                                                 _ptr(w_packed), _ptr(bias_packed), _ptr(w_fold), _ptr(cd), _ptr(out),
                                                 _ptr(status), int(timeout_ns), _stream())
    _lib.check(rc, "trimul_sm100_forward_static")


def peer_signal(flag_peer_ptrs: Sequence[int], slot: int) -> None:
    """Add 1 to counter ``slot`` on every rank of the cp group (enqueued on the current stream)."""
    rc = _lib.load().trimul_sm100_peer_signal(_ptr_array(flag_peer_ptrs), len(flag_peer_ptrs), int(slot), _stream())
    _lib.check(rc, "trimul_sm100_peer_signal")


def peer_wait(local_flags: torch.Tensor, slot: int, expected: int, status, timeout_ns: int = DEFAULT_TIMEOUT_NS,
              timeline: Optional[torch.Tensor] = None) -> None:
    """Hold the current stream until this rank's counter ``slot`` reaches ``expected`` (bounded)."""
    rc = _lib.load().trimul_sm100_peer_wait(_ptr(local_flags), int(slot), int(expected), _ptr(status),
                                            _ptr(timeline), int(timeout_ns), _stream())
    _lib.check(rc, "trimul_sm100_peer_wait")


class Plan:
    """One rank's three launches for a fixed geometry and set of buffers (``trimul_plan_t``): every TMA
    descriptor is encoded once here instead of on every forward.  Holds references to the tensors whose
    addresses it captured; ``close()`` (or garbage collection) releases the host object."""

    def __init__(self, geom, weights, ab_peer_ptrs: Sequence[int], tri_peer_ptrs: Sequence[int], gate: torch.Tensor,
                 status: torch.Tensor, *, timeline: Optional[torch.Tensor] = None, timeout_ns: int = DEFAULT_TIMEOUT_NS,
                 tuning=None):
        _require(gate, torch.bfloat16, "gate")
        d = _lib.PlanDesc()
        d.geom = geom
        d.tuning = tuning if tuning is not None else _lib.Tuning()
        d.ln_in_w, d.ln_in_b = _ptr(weights.norm_in_w), _ptr(weights.norm_in_b)
        d.w_packed, d.bias_packed = _ptr(weights.w_packed), _ptr(weights.bias_packed)
        d.w_fold, d.cd = _ptr(weights.w_fold), _ptr(weights.cd)
        for i, p in enumerate(ab_peer_ptrs):
            d.ab_peers[i] = int(p)
        for i, p in enumerate(tri_peer_ptrs):
            d.tri_peers[i] = int(p)
        d.gate, d.status, d.timeline, d.timeout_ns = _ptr(gate), _ptr(status), _ptr(timeline), int(timeout_ns)
        self._keep = (weights, gate, status, timeline)
        handle = C.c_void_p()
        _lib.check(_lib.load().trimul_sm100_plan_create(C.byref(d), C.byref(handle)), "trimul_sm100_plan_create")
        self._h = handle

    def ln_gated_proj(self, x: torch.Tensor, mask: Optional[torch.Tensor]) -> None:
        _require(x, torch.bfloat16, "x")
        mptr, mkind = _mask_args(mask)
        _lib.check(_lib.load().trimul_sm100_plan_ln_gated_proj(self._h, _ptr(x), mptr, mkind, _stream()),
                   "trimul_sm100_plan_ln_gated_proj")

    def tri_contract(self) -> None:
        _lib.check(_lib.load().trimul_sm100_plan_tri_contract(self._h, _stream()), "trimul_sm100_plan_tri_contract")

    def ln_out_proj(self, out: torch.Tensor) -> None:
        _require(out, torch.bfloat16, "out")
        _lib.check(_lib.load().trimul_sm100_plan_ln_out_proj(self._h, _ptr(out), _stream()),
                   "trimul_sm100_plan_ln_out_proj")

    def close(self) -> None:
        if self._h is not None and self._h.value:
            _lib.load().trimul_sm100_plan_destroy(self._h)
        self._h = None

    def __del__(self):  # pragma: no cover - interpreter teardown order
        try:
            self.close()
        except Exception:
            pass
