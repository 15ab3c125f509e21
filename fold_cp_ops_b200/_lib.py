"""ctypes binding of ``libtrimul_sm100.so`` (C ABI declared in ``include/trimul_sm100.h``).

There is exactly one compute path: the hand-written sm_100a kernels in that library.  If the
library is missing or the device is not compute capability 10.x the functions here raise; nothing
falls back to PyTorch or to the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
LIB_NAME = "libtrimul_sm100.so"

TRIMUL_OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_UNSUPPORTED_ARCH = -2
ERR_CUDA = -3
ERR_UNSUPPORTED_SHAPE = -4

MASK_NONE, MASK_BF16, MASK_FP32, MASK_U8 = 0, 1, 2, 3
OUTGOING, INCOMING = 0, 1
MAX_PEERS = 8
STATIC_SCRATCH_BYTES = 32 << 20

#: every symbol include/trimul_sm100.h declares; the CPU test-suite checks the library exports them
EXPORTED_SYMBOLS = (
    "trimul_sm100_query",
    "trimul_sm100_workspace",
    "trimul_sm100_reshard_plan",
    "trimul_sm100_contract_walk",
    "trimul_sm100_last_error",
    "trimul_sm100_build_id",
    "trimul_sm100_pack_weights",
    "trimul_sm100_pack_out_weights",
    "trimul_sm100_ln_gated_proj",
    "trimul_sm100_tri_contract",
    "trimul_sm100_ln_out_proj",
    "trimul_sm100_forward",
    "trimul_sm100_forward_static",
    "trimul_sm100_plan_create",
    "trimul_sm100_plan_ln_gated_proj",
    "trimul_sm100_plan_tri_contract",
    "trimul_sm100_plan_ln_out_proj",
    "trimul_sm100_plan_destroy",
    "trimul_sm100_peer_signal",
    "trimul_sm100_peer_wait",
)


class Caps(C.Structure):
    _fields_ = [("cc_major", C.c_int32), ("cc_minor", C.c_int32), ("num_sms", C.c_int32),
                ("max_smem_per_block", C.c_int32), ("supported", C.c_int32)]


class Geom(C.Structure):
    _fields_ = [("batch", C.c_int32), ("n", C.c_int32), ("d", C.c_int32), ("cp0", C.c_int32),
                ("cp1", C.c_int32), ("rank", C.c_int32), ("direction", C.c_int32), ("eps", C.c_float)]


class Tuning(C.Structure):
    _fields_ = [("contract_form", C.c_int32), ("front_fixed_order", C.c_int32),
                ("contract_band_rows", C.c_int32), ("contract_fixed_start", C.c_int32),
                ("contract_pace_ns", C.c_int32), ("reserved", C.c_int32 * 3)]


CONTRACT_DEFAULT, CONTRACT_SINGLE, CONTRACT_PAIR = 0, 1, 2
TIMELINE_SLOTS = 16
TL_FRONT_START, TL_FRONT_FIRST_STORE, TL_FRONT_LAST_STORE = 0, 1, 2
TL_CONTRACT_START, TL_CONTRACT_LAST_STORE, TL_OUT_START, TL_OUT_END, TL_WAIT_BASE = 3, 4, 5, 6, 8


class Status(C.Structure):
    _fields_ = [("code", C.c_int32), ("kernel", C.c_int32), ("block", C.c_int32), ("role", C.c_int32),
                ("detail", C.c_int32), ("pad", C.c_int32 * 3)]


class PlanDesc(C.Structure):
    _fields_ = [("geom", Geom), ("tuning", Tuning), ("ln_in_w", C.c_void_p), ("ln_in_b", C.c_void_p),
                ("w_packed", C.c_void_p), ("bias_packed", C.c_void_p), ("w_fold", C.c_void_p), ("cd", C.c_void_p),
                ("ab_peers", C.c_void_p * MAX_PEERS), ("tri_peers", C.c_void_p * MAX_PEERS), ("gate", C.c_void_p),
                ("status", C.c_void_p), ("timeline", C.c_void_p), ("timeout_ns", C.c_uint64)]


class Workspace(C.Structure):
    _fields_ = [("ab_bytes", C.c_uint64), ("tri_bytes", C.c_uint64), ("gate_bytes", C.c_uint64)]


class ReshardPlan(C.Structure):
    _fields_ = [("n_lines", C.c_int32), ("n_walk", C.c_int32), ("batch_rows", C.c_int64), ("line_rows", C.c_int64),
                ("walk_rows", C.c_int64), ("plane_elems", C.c_int64), ("dst_base", C.c_int64), ("dst_line", C.c_int64),
                ("d_loc", C.c_int32), ("planes", C.c_int32), ("ni_loc", C.c_int32), ("nj_loc", C.c_int32),
                ("chan_offset", C.c_int32), ("pad", C.c_int32), ("rows", C.c_int64)]


class TrimulLibraryError(RuntimeError):
    """The native library is missing, cannot be loaded, or a call into it failed."""


_lock = threading.Lock()
_lib = None


def library_path() -> Path:
    override = os.environ.get("CPO_TRIMUL_LIB")
    return Path(override) if override else _PKG_DIR / LIB_NAME


def _stale_reason(lib) -> str:
    """'' when the library was compiled from the sources beside it (or there are none to compare with)."""
    if os.environ.get("CPO_TRIMUL_LIB") or not (_PKG_DIR / "csrc").is_dir():
        return ""
    lib.trimul_sm100_build_id.restype = C.c_char_p
    lib.trimul_sm100_build_id.argtypes = []
    built_from = lib.trimul_sm100_build_id().decode()
    from .build import source_digest

    have = source_digest()
    return "" if built_from == have else f"library build id {built_from}, sources {have}"


def load():
    """Load the shared library once; raise :class:`TrimulLibraryError` if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path()
        if not path.exists():
            raise TrimulLibraryError(
                f"{path} not found. Build it with `python -m fold_cp_ops_b200.build` (needs nvcc); "
                "there is no PyTorch or CPU fallback for the TriMul kernels."
            )
        try:
            lib = C.CDLL(str(path))
        except OSError as exc:  # pragma: no cover - depends on the host
            raise TrimulLibraryError(f"cannot load {path}: {exc}") from exc
        missing = [name for name in EXPORTED_SYMBOLS if not hasattr(lib, name)]
        if missing:
            raise TrimulLibraryError(
                f"{path} was built from older sources: it does not export {missing}. Rebuild it with "
                "`python -m fold_cp_ops_b200.build`.")
        stale = _stale_reason(lib)
        if stale:
            raise TrimulLibraryError(
                f"{path} was not built from the CUDA sources next to it ({stale}); rebuild it with "
                "`python -m fold_cp_ops_b200.build` (a stale library is never loaded silently).")
        vp, i32, u64, f32p = C.c_void_p, C.c_int32, C.c_uint64, C.c_void_p
        lib.trimul_sm100_last_error.restype = C.c_char_p
        lib.trimul_sm100_last_error.argtypes = []
        lib.trimul_sm100_query.argtypes = [C.c_int, C.POINTER(Caps)]
        lib.trimul_sm100_workspace.argtypes = [C.POINTER(Geom), C.POINTER(Workspace)]
        lib.trimul_sm100_reshard_plan.argtypes = [C.POINTER(Geom), C.POINTER(ReshardPlan)]
        lib.trimul_sm100_reshard_plan.restype = C.c_int
        lib.trimul_sm100_contract_walk.argtypes = [C.POINTER(Geom), C.POINTER(Tuning), C.c_int32, C.POINTER(C.c_int32),
                                                   C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
        lib.trimul_sm100_contract_walk.restype = C.c_int
        lib.trimul_sm100_pack_weights.argtypes = [i32, vp, vp, vp, f32p, f32p, f32p, vp, f32p, vp]
        lib.trimul_sm100_ln_gated_proj.argtypes = [C.POINTER(Geom), C.POINTER(Tuning), vp, vp, i32, f32p, f32p, vp, f32p,
                                                   C.POINTER(vp), vp, vp, u64, vp]
        lib.trimul_sm100_tri_contract.argtypes = [C.POINTER(Geom), C.POINTER(Tuning), vp, C.POINTER(vp), vp, u64, vp]
        lib.trimul_sm100_plan_create.argtypes = [C.POINTER(PlanDesc), C.POINTER(vp)]
        lib.trimul_sm100_plan_ln_gated_proj.argtypes = [vp, vp, vp, i32, vp]
        lib.trimul_sm100_plan_tri_contract.argtypes = [vp, vp]
        lib.trimul_sm100_plan_ln_out_proj.argtypes = [vp, vp, vp]
        lib.trimul_sm100_plan_destroy.argtypes = [vp]
        lib.trimul_sm100_plan_destroy.restype = None
        lib.trimul_sm100_pack_out_weights.argtypes = [i32, vp, f32p, f32p, f32p, vp, f32p, vp]
        lib.trimul_sm100_ln_out_proj.argtypes = [C.POINTER(Geom), vp, vp, vp, f32p, vp, vp, u64, vp]
        lib.trimul_sm100_forward.argtypes = [C.POINTER(Geom), vp, vp, i32, f32p, f32p, vp, f32p, vp, f32p,
                                             vp, vp, vp, vp, vp, u64, vp]
        lib.trimul_sm100_forward_static.argtypes = [C.POINTER(Geom), vp, vp, i32, f32p, f32p, vp, f32p, vp, f32p,
                                                    vp, vp, u64, vp]
        lib.trimul_sm100_forward_static.restype = C.c_int
        lib.trimul_sm100_peer_signal.argtypes = [C.POINTER(vp), i32, i32, vp]
        lib.trimul_sm100_peer_wait.argtypes = [vp, i32, u64, vp, vp, u64, vp]
        for name in ("trimul_sm100_query", "trimul_sm100_workspace", "trimul_sm100_pack_weights",
                     "trimul_sm100_pack_out_weights",
                     "trimul_sm100_ln_gated_proj", "trimul_sm100_tri_contract", "trimul_sm100_ln_out_proj",
                     "trimul_sm100_forward", "trimul_sm100_peer_signal", "trimul_sm100_peer_wait",
                     "trimul_sm100_plan_create", "trimul_sm100_plan_ln_gated_proj", "trimul_sm100_plan_tri_contract",
                     "trimul_sm100_plan_ln_out_proj"):
            getattr(lib, name).restype = C.c_int
        _lib = lib
        return lib


def last_error() -> str:
    return load().trimul_sm100_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc == TRIMUL_OK:
        return
    msg = last_error()
    if rc == ERR_UNSUPPORTED_SHAPE or rc == ERR_INVALID_ARGUMENT:
        raise ValueError(f"{what}: {msg}")
    raise TrimulLibraryError(f"{what} failed (code {rc}): {msg}")
