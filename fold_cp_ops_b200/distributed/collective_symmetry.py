"""Group-uniform decisions and bounded barriers.

Public surface of the reference's ``fold_cp_ops/distributed/collective_symmetry.py:113-365``:
``CollectiveGate`` (``agree_bool``, ``barrier``, ``guard``, ``should_skip``) and the exception
family ``CollectiveError`` > ``CollectiveFailure`` / ``PeerFailure`` / ``BarrierTimeout``.  The
rule they enforce: a decision one rank could make differently from its peers (an exception, a
skip, an out-of-memory) is reduced over the group BEFORE anyone acts on it, so ranks leave a
collective region together or not at all.  Works on any backend (NCCL on GPUs, gloo on CPUs).
"""
from __future__ import annotations

import contextlib
import datetime
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

__all__ = ["CollectiveGate", "CollectiveError", "CollectiveFailure", "PeerFailure", "BarrierTimeout",
           "DEFAULT_BARRIER_TIMEOUT_S"]

DEFAULT_BARRIER_TIMEOUT_S = float(os.environ.get("CPO_BARRIER_TIMEOUT_S", "480"))
_POLL_S = 0.05


class CollectiveError(RuntimeError):
    """The group disagreed (base class)."""


class CollectiveFailure(CollectiveError):
    """This rank's own guarded block failed; chained to the original exception."""


class PeerFailure(CollectiveError):
    """This rank's guarded block succeeded but a peer's did not; the peer's log has the cause."""


class BarrierTimeout(CollectiveError):
    """A bounded barrier did not complete within its bound."""


class CollectiveGate:
    """One per process group.  Every method is COLLECTIVE: all ranks must reach it, in order."""

    def __init__(self, group=None, device=None, timeout_s: float = DEFAULT_BARRIER_TIMEOUT_S):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError(
                "CollectiveGate needs an initialized torch.distributed process group; call "
                "init_process_group first. Constructing it earlier hides the real error behind a "
                "collective failure several frames later.")
        self.group = group
        self.timeout_s = timeout_s
        if device is None:
            backend = dist.get_backend(group)
            if "nccl" in str(backend) and torch.cuda.is_available():
                device = torch.device("cuda", torch.cuda.current_device())
            else:
                device = torch.device("cpu")
        self.device = torch.device(device)

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group)

    def agree_bool(self, local: bool, *, op: str = "any") -> bool:
        """``"any"``: true if any rank passed True; ``"all"``: only if every rank did."""
        if op not in ("any", "all"):
            raise ValueError(f"op must be 'any' or 'all'; got {op!r}")
        t = torch.tensor([1.0 if local else 0.0], device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "any" else dist.ReduceOp.MIN, group=self.group)
        return bool(t.item() > 0)

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        """Barrier that raises :class:`BarrierTimeout` instead of waiting forever.

        ``CPO_BARRIER_WAIT`` selects how the wait is done: ``poll`` (default; poll the async work
        handle), ``wait`` (``work.wait(timeout)``), ``sync`` (plain blocking barrier, unbounded)."""
        bound = self.timeout_s if timeout_s is None else timeout_s
        if bound <= 0:
            raise ValueError(f"barrier timeout must be positive; got {bound}")
        mode = os.environ.get("CPO_BARRIER_WAIT", "poll")
        if mode == "sync":
            if self.device.type == "cuda":
                dist.barrier(group=self.group, device_ids=[self.device.index])
            else:
                dist.barrier(group=self.group)
            return
        work = dist.barrier(group=self.group, async_op=True)
        if work is None:
            return
        gone = (f"rank {self.rank} waited {bound:.0f}s at a collective barrier and at least one peer never "
                "arrived. The group is now desynchronized -- do NOT enter another collective. A peer has died, "
                "hung, or taken a divergent path (a per-rank skip or an unguarded exception are the usual causes).")
        if mode == "wait":
            try:
                done = work.wait(timeout=datetime.timedelta(seconds=bound))
            except Exception as exc:  # noqa: BLE001 - any failure here means the bound was not honoured
                raise BarrierTimeout(gone) from exc
            if done is False:
                raise BarrierTimeout(gone)
            return
        deadline = time.monotonic() + bound
        while not work.is_completed():
            if time.monotonic() > deadline:
                raise BarrierTimeout(gone)
            time.sleep(_POLL_S)

    @contextlib.contextmanager
    def guard(self, what: str):
        """A failure inside the block on ANY rank raises on EVERY rank, after one reduction."""
        held: Optional[BaseException] = None
        try:
            yield
        except BaseException as exc:  # noqa: BLE001 - re-raised after the reduction
            held = exc
        if not self.agree_bool(held is not None, op="any"):
            return
        if held is not None:
            raise CollectiveFailure(
                f"[{what}] failed on rank {self.rank} (surfaced collectively so no rank proceeds alone): "
                f"{type(held).__name__}: {held}") from held
        raise PeerFailure(
            f"[{what}] succeeded on rank {self.rank} but FAILED on at least one peer, so this rank stops here "
            "rather than entering the next collective alone. The failing rank's log holds the original traceback.")

    def should_skip(self, local_reason: Optional[str]) -> Optional[str]:
        """Skip together or not at all: returns the agreed reason, or ``None`` to proceed."""
        if not self.agree_bool(local_reason is not None, op="any"):
            return None
        return local_reason or "a peer rank requested a skip (this rank's own predicate passed)"
