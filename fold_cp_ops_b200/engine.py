"""The TriMul engine: weights, workspaces and the three-kernel chain for one rank.

Takes over the job of the reference's ``TriMulAutotuned``
(``fold_cp_ops/distributed/workflows/trimul_autotuned.py:2646-3763``): it owns the packed
weights, the operand / result buffers (symmetric across the cp group when cp > 1) and runs

    ln_gated_proj  ->  [front flags]  ->  tri_contract  ->  [back flags]  ->  ln_out_proj

on the current CUDA stream.  There is no NCCL call, no host synchronisation and no separate
all-to-all on that path: the two reshards are the kernels' own epilogue stores into the owning
rank's buffer, and rank-to-rank ordering is a counter exchange done by two tiny flag kernels.
At cp=1 the same kernels run with a one-entry peer table and no flag kernels at all.

Every launch goes through a :class:`fold_cp_ops_b200.kernels.Plan` that is built once per
``(B, N, direction)`` -- the TMA descriptors of a forward are encoded when the workspace is made,
not on every call.

A device-side wait that expires makes its kernel return early and leaves a status record.  The
engine copies that record to pinned host memory after every forward; the NEXT forward (and
:meth:`TriMulEngine.check`) raises :class:`DeviceWaitTimeout` when it finds one, so a caller of the
public API cannot keep consuming outputs of a forward that gave up.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from . import kernels as K

SUPPORTED_D = (128, 256, 384, 512)

#: default bound of the cross-rank flag waits.  Much longer than the in-kernel pipeline waits (2 s):
#: a peer whose HOST is late (data loading, checkpoint IO, garbage collection) must be waited for, as
#: the reference's drains do; the bound only exists so that a dead peer cannot hang a shared GPU.
DEFAULT_PEER_TIMEOUT_NS = 30_000_000_000

#: measured defaults of the sm_100a kernels per (feature width, cp): form of the contraction kernel and
#: whether the projection kernel's CTAs walk their gated chunks in rotated order.  CTA pairs won at
#: every shape (27.5 vs 30.8 ms at N=4096 D=256, 3.13 vs 3.45 ms at N=2048); the rotation costs nothing
#: at cp=1 and spreads the peer stores over all NVLink directions at cp>1 (cp=2: 9.1-9.4 vs 9.7-10.3 ms).
#: The contraction's tile walk (bands of 8 tile rows, own-block start) and the pacing of its CTA pairs (20 us)
#: are the library's own defaults (a zero in the tuning record); an entry here may override them per (D, cp)
#: with "contract_band_rows" / "contract_pace_ns".
SM100_DEFAULTS = {(d, cp): {"contract_form": "pair", "front_fixed_order": False}
                  for d in SUPPORTED_D for cp in (1, 2, 4, 8)}


def _env_ms(name: str) -> Optional[int]:
    v = os.environ.get(name)
    return int(float(v) * 1e6) if v else None


@dataclass
class CpGeometry:
    """How the (N, N) token grid is split over the cp group and where this rank sits.

    ``cp0`` splits rows (tensor dim 1), ``cp1`` columns (tensor dim 2); ``rank`` is this rank's
    index in row-major (row block, column block) order; ``peers[r]`` is the global rank of the
    member at that index."""

    cp0: int = 1
    cp1: int = 1
    rank: int = 0
    peers: Tuple[int, ...] = (0,)

    @property
    def cp(self) -> int:
        return self.cp0 * self.cp1


class PackedWeights:
    """Device-resident weights in the form the kernels read (built once per layer).

    LayerNorm gains / biases and projection biases stay fp32; the six projection matrices are
    bf16; the three input-side matrices are regrouped into the five chunk order of
    ``trimul_sm100_pack_weights`` (pre-scaled by 1/2); the output LayerNorm is folded into the output
    projection by ``trimul_sm100_pack_out_weights``."""

    def __init__(self, w: Dict[str, Optional[torch.Tensor]], device: torch.device):
        D = int(w["norm_in_w"].shape[0])
        if D not in SUPPORTED_D:
            raise ValueError(f"feature width D={D} is not supported by the sm_100a kernels (supported: {SUPPORTED_D})")
        for key, shape in (("p_in_w", (2 * D, D)), ("g_in_w", (2 * D, D)), ("p_out_w", (D, D)), ("g_out_w", (D, D))):
            if tuple(w[key].shape) != shape:
                raise ValueError(f"{key} must be {shape}; got {tuple(w[key].shape)}")
        self.D = D
        f32 = lambda t: None if t is None else t.detach().to(device=device, dtype=torch.float32).contiguous()
        b16 = lambda t: t.detach().to(device=device, dtype=torch.bfloat16).contiguous()
        self.norm_in_w, self.norm_in_b = f32(w["norm_in_w"]), f32(w.get("norm_in_b"))
        # the output LayerNorm is folded into the output projection: bf16(gamma * W) and (c, d) constants
        self.w_fold, self.cd = K.pack_out_weights(D, b16(w["p_out_w"]), f32(w["norm_out_w"]), f32(w.get("norm_out_b")),
                                                  f32(w.get("p_out_b")))
        self.w_packed, self.bias_packed = K.pack_weights(
            D, b16(w["p_in_w"]), b16(w["g_in_w"]), b16(w["g_out_w"]), f32(w.get("p_in_b")), f32(w.get("g_in_b")),
            f32(w.get("g_out_b")))
        if all(w.get(k) is None for k in ("p_in_b", "g_in_b", "g_out_b")):
            self.bias_packed = None  # lets the projection kernel skip every bias load


class TriMulEngine:
    """One rank's fused TriMul forward.

    ``forward(x_local, direction, mask_local)`` takes this rank's ``(B, N/cp0, N/cp1, D)`` block
    and returns the same block of the output, freshly allocated, bf16.  Workspaces are cached per
    ``(B, N)``; at cp > 1 they are symmetric allocations exchanged once with the peers.

    Tuning (all optional): ``contract_form`` ``"auto" | "single" | "pair"``, ``front_fixed_order``,
    ``contract_band_rows`` (tile rows per band of the contraction's tile walk; 0 = the library's choice),
    ``contract_fixed_start`` (every rank walks the contraction's tiles from tile (0, 0)),
    ``contract_pace_ns`` (longest wait of a CTA pair for the others before a tile; 0 = the library's choice,
    negative = off),
    ``wait_timeout_ms`` (bound of the cross-rank flag waits; ``CPO_A2A_WAIT_TIMEOUT_MS`` overrides).
    """

    def __init__(self, w: Dict[str, Optional[torch.Tensor]], *, device: torch.device, eps: float = 1e-5,
                 geometry: Optional[CpGeometry] = None, process_group=None, recv_cache: Optional[int] = None,
                 contract_form: Optional[str] = None, front_fixed_order: Optional[bool] = None,
                 contract_band_rows: Optional[int] = None, contract_fixed_start: Optional[bool] = None,
                 contract_pace_ns: Optional[int] = None, wait_timeout_ms: Optional[float] = None):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("TriMulEngine needs a CUDA device: the TriMul kernels have no CPU path")
        K.device_caps(self.device.index if self.device.index is not None else torch.cuda.current_device())
        with torch.cuda.device(self.device):
            self.weights = PackedWeights(w, self.device)
        self.D = self.weights.D
        self.eps = float(eps)
        self.geometry = geometry or CpGeometry()
        self.group = process_group
        if self.geometry.cp > 1 and process_group is None:
            raise ValueError("a cp > 1 engine needs the process group of its cp peers")
        defaults = SM100_DEFAULTS.get((self.D, self.geometry.cp), {"contract_form": "auto", "front_fixed_order": False})
        self.contract_form = contract_form if contract_form is not None else defaults["contract_form"]
        self.front_fixed_order = bool(defaults["front_fixed_order"] if front_fixed_order is None else front_fixed_order)
        self.contract_band_rows = int(defaults.get("contract_band_rows", 0) if contract_band_rows is None else contract_band_rows)
        self.contract_fixed_start = bool(contract_fixed_start)
        self.contract_pace_ns = int(defaults.get("contract_pace_ns", 0) if contract_pace_ns is None else contract_pace_ns)
        self.tuning = K.make_tuning(self.contract_form, self.front_fixed_order, self.contract_band_rows,
                                    self.contract_fixed_start, self.contract_pace_ns)
        self.status = K.new_status(self.device)
        self._status_host = torch.zeros(8, dtype=torch.int32).pin_memory()
        self._status_event: Optional[torch.cuda.Event] = None
        self.timeout_ns = K.DEFAULT_TIMEOUT_NS
        env_wait = _env_ms("CPO_A2A_WAIT_TIMEOUT_MS")
        self.peer_timeout_ns = env_wait or (int(wait_timeout_ms * 1e6) if wait_timeout_ms else DEFAULT_PEER_TIMEOUT_NS)
        cap = os.environ.get("CPO_TRIMUL_RECV_CACHE")
        self._cache_cap = int(cap) if cap else (recv_cache if recv_cache is not None else 2)
        self._ws: Dict[Tuple[int, int], "_Workspace"] = {}
        self.stage_log = bool(int(os.environ.get("CPO_TRIMUL_STAGE_LOG", "0") or 0))
        self.collect_stats = self.stage_log
        self.last_stage_ms: Dict[str, float] = {}
        self._last_stats: Dict[str, object] = {}
        self._stats_ws: Optional["_Workspace"] = None

    # ------------------------------------------------------------------------------------------
    def _check_shapes(self, x_local: torch.Tensor, N: int) -> None:
        g = self.geometry
        cp = g.cp
        if self.D % cp != 0:
            raise ValueError(f"D={self.D} must be divisible by cp={cp}")
        if N % g.cp0 != 0 or N % g.cp1 != 0:
            raise ValueError(f"N={N} must be divisible by each cp axis {(g.cp0, g.cp1)}")
        if N % 8 != 0:
            raise ValueError(f"N must be 16-byte aligned (N % 8 == 0 for a 16-bit activation); got N={N}")
        if cp > 1 and ((N // g.cp0) % 8 != 0 or (N // g.cp1) % 8 != 0):
            raise ValueError(f"local token extents {(N // g.cp0, N // g.cp1)} must be multiples of 8")
        want = (N // g.cp0, N // g.cp1, self.D)
        if tuple(x_local.shape[1:]) != want:
            raise ValueError(f"x_local must be (B, {want[0]}, {want[1]}, {want[2]}); got {tuple(x_local.shape)}")

    def _workspace(self, B: int, N: int) -> "_Workspace":
        key = (B, N)
        ws = self._ws.get(key)
        if ws is None:
            while len(self._ws) >= max(1, self._cache_cap):
                self._ws.pop(next(iter(self._ws))).close()  # FIFO; buffers return to their pool by refcount
            ws = _Workspace(self, B, N)
            self._ws[key] = ws
        return ws

    def prepare(self, B: int, N: int) -> None:
        """Allocate (and, at cp > 1, exchange) the buffers for this shape ahead of the first forward."""
        with torch.cuda.device(self.device):
            self._workspace(int(B), int(N))

    @torch.no_grad()
    def forward(self, x_local: torch.Tensor, direction: str, mask_local: Optional[torch.Tensor] = None) -> torch.Tensor:
        if direction not in ("outgoing", "incoming"):
            raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}")
        if x_local.dim() != 4:
            raise ValueError(f"x_local must be (B, N_i, N_j, D); got {tuple(x_local.shape)}")
        g = self.geometry
        B = int(x_local.shape[0])
        N = int(x_local.shape[1]) * g.cp0
        self._check_shapes(x_local, N)
        if x_local.device != self.device:
            raise ValueError(f"x_local is on {x_local.device}, the engine on {self.device}")
        self._raise_if_previous_forward_gave_up()
        x = x_local if x_local.dtype is torch.bfloat16 else x_local.to(torch.bfloat16)
        x = x.contiguous()
        mask = None
        if mask_local is not None:
            if tuple(mask_local.shape) != tuple(x.shape[:3]) and mask_local.numel() != x.shape[0] * x.shape[1] * x.shape[2]:
                raise ValueError(f"mask must be {tuple(x.shape[:3])}; got {tuple(mask_local.shape)}")
            mask = mask_local
            if mask.dtype not in (torch.bfloat16, torch.float32, torch.uint8, torch.bool):
                mask = mask.to(torch.float32)
            mask = mask.contiguous()
        with torch.cuda.device(self.device):
            ws = self._workspace(B, N)
            out = torch.empty_like(x)
            ws.run(x, mask, direction, out)
            # mirror the status record to the host: read by the next forward / check() without a sync
            self._status_host.copy_(self.status, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._status_event = ev
        return out

    # ------------------------------------------------------------------------------------------
    def _raise_from(self, record) -> None:
        self.status.zero_()
        self._status_host.zero_()
        self._status_event = None
        raise K.DeviceWaitTimeout(K.describe_status(record))

    def _raise_if_previous_forward_gave_up(self) -> None:
        """Non-blocking: looks at the host mirror of the status record if its copy has finished."""
        ev = self._status_event
        if ev is not None and ev.query():
            rec = self._status_host.tolist()
            if rec[0] != 0:
                self._raise_from(rec)

    def check(self) -> None:
        """Synchronising check of the device status record: raises :class:`DeviceWaitTimeout` if any
        bounded wait of a forward issued so far expired (that forward's output is invalid)."""
        rec = self.status.tolist()
        if rec[0] != 0:
            self._raise_from(rec)

    def last_forward_stats(self) -> Dict[str, object]:
        """Measurements of the most recent forward made with ``collect_stats = True`` (synchronises).

        ``stage_ms``: CUDA-event time of the three kernels alone (the flag kernels are outside these
        windows); ``wait_ms``: time this rank's stream sat in each cross-rank flag wait, from the
        device timeline (the all-to-all time that was NOT hidden behind a kernel); ``span_ms``:
        first-CTA-start to last-store of each kernel on the device clock; ``bytes_to_peers``: bytes
        this rank's epilogues stored into other ranks' buffers."""
        ws = self._stats_ws
        if ws is None:
            return dict(self._last_stats)
        self._last_stats = ws.collect()
        self._stats_ws = None
        return dict(self._last_stats)

    def free(self) -> None:
        """Drop the cached workspaces.  Symmetric blocks go back to their pool by refcount; no
        collective runs here, so ranks may call this in any order."""
        for ws in self._ws.values():
            ws.close()
        self._ws.clear()


_TL_FIRST = (_lib.TL_FRONT_START, _lib.TL_FRONT_FIRST_STORE, _lib.TL_CONTRACT_START, _lib.TL_OUT_START)


class _Workspace:
    """Buffers and launch plans for one ``(B, N)``.  cp=1: plain allocations, optionally one batch
    plane at a time when the full-batch operand buffer would not fit; cp>1: symmetric allocations +
    flag pads."""

    def __init__(self, eng: TriMulEngine, B: int, N: int):
        self.eng, self.B, self.N = eng, B, N
        g = eng.geometry
        D = eng.D
        dev = eng.device
        self.ni, self.nj = N // g.cp0, N // g.cp1
        self.planes_b = B  # batch planes handled per kernel launch
        self.timeline = torch.zeros(_lib.TIMELINE_SLOTS, dtype=torch.int64, device=dev)
        preset = torch.zeros(_lib.TIMELINE_SLOTS, dtype=torch.int64)
        preset[list(_TL_FIRST)] = -1  # all ones: the identity of an unsigned min
        self._tl_preset = preset.to(dev)
        if g.cp == 1:
            geom = K.make_geom(B, N, D, "outgoing", eng.eps)
            need = K.workspace_bytes(geom)
            total = need.ab_bytes + need.tri_bytes + need.gate_bytes
            free, _ = torch.cuda.mem_get_info(dev)
            budget = int(os.environ.get("CPO_TRIMUL_WORKSPACE_BYTES", 0)) or int(free * 0.9)
            if B > 1 and total + 2 * B * N * N * D > budget:
                self.planes_b = 1
            pb = self.planes_b
            self.ab = torch.empty((2, D, pb, N, N), dtype=torch.bfloat16, device=dev)
            self.tri = torch.empty((D, pb, N, N), dtype=torch.bfloat16, device=dev)
            self.gate = torch.empty((pb, N, N, D), dtype=torch.bfloat16, device=dev)
            self.ab_ptrs = [self.ab.data_ptr()]
            self.tri_ptrs = [self.tri.data_ptr()]
            self.flags = None
        else:
            from .distributed import symmetric

            d_loc = D // g.cp
            self.sym = symmetric.SymmetricWorkspace(
                eng.group, dev, g, ab_shape=(2, d_loc, B, N, N), tri_shape=(D, B, self.ni, self.nj),
                status=eng.status, timeout_ns=eng.peer_timeout_ns, timeline=self.timeline)
            self.ab, self.tri = self.sym.ab, self.sym.tri
            self.ab_ptrs, self.tri_ptrs = self.sym.ab_ptrs, self.sym.tri_ptrs
            self.gate = torch.empty((B, self.ni, self.nj, D), dtype=torch.bfloat16, device=dev)
            self.flags = self.sym.flags
        self._plans: Dict[str, K.Plan] = {}
        self._events = None

    def _plan(self, direction: str) -> K.Plan:
        plan = self._plans.get(direction)
        if plan is None:
            eng, g = self.eng, self.eng.geometry
            geom = K.make_geom(self.planes_b, self.N, eng.D, direction, eng.eps, g.cp0, g.cp1, g.rank)
            plan = K.Plan(geom, eng.weights, self.ab_ptrs, self.tri_ptrs, self.gate, eng.status,
                          timeline=self.timeline, timeout_ns=eng.timeout_ns, tuning=eng.tuning)
            self._plans[direction] = plan
        return plan

    def close(self) -> None:
        for plan in self._plans.values():
            plan.close()
        self._plans.clear()

    def run(self, x, mask, direction, out) -> None:
        eng = self.eng
        pb = self.planes_b
        stats = eng.collect_stats or eng.stage_log
        plan = self._plan(direction)
        for b0 in range(0, self.B, pb):
            xs = x[b0:b0 + pb]
            ms = None if mask is None else mask.reshape(self.B, self.ni, self.nj)[b0:b0 + pb]
            os_ = out[b0:b0 + pb]
            ev = None
            if stats:
                self.timeline.copy_(self._tl_preset)
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
                ev[0].record()
            plan.ln_gated_proj(xs, ms)
            if stats:
                ev[1].record()
            if self.flags is not None:
                self.flags.front_done()
            if stats:
                ev[2].record()
            plan.tri_contract()
            if stats:
                ev[3].record()
            if self.flags is not None:
                self.flags.back_done()
            if stats:
                ev[4].record()
            plan.ln_out_proj(os_)
            if stats:
                ev[5].record()
            if self.flags is not None:
                self.flags.consumed()
            if stats:
                self._events = ev
                eng._stats_ws = self
                if eng.stage_log:
                    eng.last_forward_stats()
                    print(f"[trimul stage log] {eng.last_stage_ms}", flush=True)

    def collect(self) -> Dict[str, object]:
        """Read the events and the device timeline of the last traced pass (synchronises)."""
        eng, g = self.eng, self.eng.geometry
        ev = self._events
        ev[5].synchronize()
        stage = {"ln_gated_proj": ev[0].elapsed_time(ev[1]), "tri_contract": ev[2].elapsed_time(ev[3]),
                 "ln_out_proj": ev[4].elapsed_time(ev[5])}
        eng.last_stage_ms = stage
        tl = self.timeline.tolist()
        ms = lambda a, b: (tl[b] - tl[a]) * 1e-6 if tl[a] > 0 and tl[b] > 0 else None
        base = _lib.TL_WAIT_BASE
        wait = {}
        if g.cp > 1:
            wait = {"front": ms(base + 0, base + 1), "back": ms(base + 2, base + 3), "consumed": ms(base + 4, base + 5)}
        span = {"ln_gated_proj": ms(_lib.TL_FRONT_START, _lib.TL_FRONT_LAST_STORE),
                "first_store_after_start": ms(_lib.TL_FRONT_START, _lib.TL_FRONT_FIRST_STORE),
                "tri_contract": ms(_lib.TL_CONTRACT_START, _lib.TL_CONTRACT_LAST_STORE),
                "ln_out_proj": ms(_lib.TL_OUT_START, _lib.TL_OUT_END),
                "forward": ms(_lib.TL_FRONT_START, _lib.TL_OUT_END)}
        s = self.planes_b * self.ni * self.nj * eng.D * 2  # bytes of one local activation
        peers = g.cp - 1
        return {"stage_ms": stage, "wait_ms": wait, "span_ms": span,
                "step_ms": ev[0].elapsed_time(ev[5]),
                "bytes_to_peers": {"front": 2 * s * peers // g.cp, "back": s * peers // g.cp}}
