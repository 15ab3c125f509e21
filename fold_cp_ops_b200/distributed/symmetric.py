"""Symmetric (peer-mapped) buffers and the flag protocol of the two fused reshards.

Takes over ``_symmetric_empty`` / ``_refuse_unsatisfiable_symmetric_request`` / ``_symmetric_free``
(``fold_cp_ops/distributed/workflows/trimul_autotuned.py:150-319``) and the barrier / drain calls
around the two all-to-alls (``:3272-3300``).

Buffers come from ``torch.distributed._symmetric_memory`` (cuMem allocations whose handles are
exchanged once over the process group); each rank then holds, for every peer, a device pointer
to that peer's copy.  The kernels store through those pointers over NVLink.

Ordering uses three monotonically increasing counters per rank (slot numbers below).  In forward
number ``e`` (1-based) of one workspace, with ``cp`` ranks:

    ln_gated_proj(e)  stores a|b into every peer          then signal FRONT on every rank
    wait FRONT >= cp*e       (every peer's a|b for forward e has landed here)
    wait CONSUMED >= cp*(e-1) (every peer has finished reading its tri of forward e-1)
    tri_contract(e)   stores tri into every peer          then signal BACK on every rank
    wait BACK >= cp*e        (every peer's tri has landed here; also: every peer is done reading
                              its a|b, so forward e+1 may overwrite them)
    ln_out_proj(e)                                        then signal CONSUMED on every rank

Every wait is a bounded device-side poll; nothing here blocks the host.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import kernels as K

SLOT_FRONT, SLOT_BACK, SLOT_CONSUMED = 0, 1, 2
NUM_SLOTS = 16


def refuse_unsatisfiable_request(nbytes: int, device: torch.device, group) -> None:
    """Rank-uniform out-of-memory: every rank votes whether ``nbytes`` fits; if any cannot, ALL raise
    ``torch.cuda.OutOfMemoryError`` before the collective allocation, so no rank enters it alone."""
    free, _ = torch.cuda.mem_get_info(device)
    ok = torch.tensor([1 if free > nbytes else 0], dtype=torch.int32, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
        raise torch.cuda.OutOfMemoryError(
            f"symmetric allocation of {nbytes / 2**30:.2f} GiB refused on every rank of the cp group: at least one "
            f"rank has less free device memory than that (this rank: {free / 2**30:.2f} GiB free)")


def symmetric_empty(shape: Sequence[int], dtype: torch.dtype, device: torch.device, group) -> Tuple[torch.Tensor, List[int]]:
    """Collective: allocate a peer-mapped tensor; return it and the per-group-rank device pointers."""
    import torch.distributed._symmetric_memory as symm_mem

    numel = 1
    for s in shape:
        numel *= int(s)
    refuse_unsatisfiable_request(numel * torch.empty((), dtype=dtype).element_size(), device, group)
    t = symm_mem.empty(*[int(s) for s in shape], dtype=dtype, device=device)
    hdl = symm_mem.rendezvous(t, group)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    if len(ptrs) != dist.get_world_size(group):
        raise RuntimeError(f"symmetric rendezvous returned {len(ptrs)} peer pointers for a group of "
                           f"{dist.get_world_size(group)}")
    return t, ptrs


class PeerFlags:
    """The three counters of one workspace and the enqueue helpers the engine calls."""

    def __init__(self, flags: torch.Tensor, flag_ptrs: List[int], cp: int, status: torch.Tensor, timeout_ns: int,
                 timeline: Optional[torch.Tensor] = None):
        self.flags, self.flag_ptrs, self.cp = flags, flag_ptrs, cp
        self.status, self.timeout_ns, self.timeline = status, timeout_ns, timeline
        self.epoch = 0

    def _wait(self, slot: int, expected: int) -> None:
        K.peer_wait(self.flags, slot, expected, self.status, self.timeout_ns, self.timeline)

    def front_done(self) -> None:
        self.epoch += 1
        K.peer_signal(self.flag_ptrs, SLOT_FRONT)
        self._wait(SLOT_FRONT, self.cp * self.epoch)
        if self.epoch > 1:
            self._wait(SLOT_CONSUMED, self.cp * (self.epoch - 1))

    def back_done(self) -> None:
        K.peer_signal(self.flag_ptrs, SLOT_BACK)
        self._wait(SLOT_BACK, self.cp * self.epoch)

    def consumed(self) -> None:
        K.peer_signal(self.flag_ptrs, SLOT_CONSUMED)


class SymmetricWorkspace:
    """Peer-mapped ``ab`` / ``tri`` buffers + flags for one ``(B, N)`` on one rank.  COLLECTIVE to build."""

    def __init__(self, group, device: torch.device, geometry, ab_shape, tri_shape, status: torch.Tensor = None,
                 timeout_ns: int = K.DEFAULT_TIMEOUT_NS, timeline: Optional[torch.Tensor] = None):
        self.group = group
        cp = geometry.cp
        if dist.get_world_size(group) != cp:
            raise ValueError(f"the cp process group has {dist.get_world_size(group)} ranks but the geometry says cp={cp}")
        # geometry.peers[r] is the GLOBAL rank of cp peer r; the rendezvous tables are indexed by group rank
        order = [dist.get_group_rank(group, int(g)) for g in geometry.peers]
        self.ab, ab_ptrs = symmetric_empty(ab_shape, torch.bfloat16, device, group)
        self.tri, tri_ptrs = symmetric_empty(tri_shape, torch.bfloat16, device, group)
        flags, flag_ptrs = symmetric_empty((NUM_SLOTS,), torch.int64, device, group)
        flags.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # nobody signals before every rank has zeroed its counters
        self.ab_ptrs = [ab_ptrs[i] for i in order]
        self.tri_ptrs = [tri_ptrs[i] for i in order]
        self._flag_tensor = flags
        self._flag_ptrs = [flag_ptrs[i] for i in order]
        self.flags = None
        if status is not None:
            self.bind(status, timeout_ns, timeline)

    def bind(self, status: torch.Tensor, timeout_ns: int, timeline: Optional[torch.Tensor] = None) -> "SymmetricWorkspace":
        self.flags = PeerFlags(self._flag_tensor, self._flag_ptrs, len(self._flag_ptrs), status, timeout_ns, timeline)
        return self
