"""Decisions a whole process group takes together, and a barrier that cannot wait forever.

Same public names as the reference's ``fold_cp_ops/distributed/collective_symmetry.py:113-365``
(``CollectiveGate`` with ``agree_bool`` / ``barrier`` / ``guard`` / ``should_skip``, and the
``CollectiveError`` family), written for this package.

Why it exists: ranks of one job run the same program, but some outcomes are local -- an exception,
a "this shape is not supported here", an out-of-memory.  A rank that acts on such an outcome alone
(returns early, skips, raises) leaves its peers inside the next collective waiting for a partner
that never comes.  The gate turns every such outcome into ONE small reduction first: afterwards all
ranks know whether anybody tripped, and they leave the region together.  It needs nothing but
``torch.distributed``, so it works over NCCL on GPUs and over gloo on CPUs alike.
"""
from __future__ import annotations

import datetime
import os
import time
from typing import Callable, Dict, Optional

import torch
import torch.distributed as dist

__all__ = ["CollectiveGate", "CollectiveError", "CollectiveFailure", "PeerFailure", "BarrierTimeout",
           "DEFAULT_BARRIER_TIMEOUT_S"]

DEFAULT_BARRIER_TIMEOUT_S = float(os.environ.get("CPO_BARRIER_TIMEOUT_S", "480"))


class CollectiveError(RuntimeError):
    """Root of the family: something about the group, not about this rank's own data, went wrong."""


class CollectiveFailure(CollectiveError):
    """Raised on the rank whose guarded block threw; ``__cause__`` is that exception."""


class PeerFailure(CollectiveError):
    """Raised on ranks whose guarded block was fine while a peer's threw."""


class BarrierTimeout(CollectiveError):
    """A bounded barrier ran out of time: some peer never arrived."""


# ---------------------------------------------------------------------------------------------
# three ways to wait for an asynchronous barrier; each returns True when it completed in time
# ---------------------------------------------------------------------------------------------
def _wait_by_polling(work, bound_s: float) -> bool:
    give_up_at = time.monotonic() + bound_s
    while time.monotonic() <= give_up_at:
        if work.is_completed():
            return True
        time.sleep(0.05)
    return work.is_completed()


def _wait_on_handle(work, bound_s: float) -> bool:
    try:
        return work.wait(timeout=datetime.timedelta(seconds=bound_s)) is not False
    except Exception:  # noqa: BLE001 - backends signal an expired wait by raising
        return False


_ASYNC_WAITS: Dict[str, Callable[[object, float], bool]] = {"poll": _wait_by_polling, "wait": _wait_on_handle}


class _GuardedRegion:
    """Context manager behind :meth:`CollectiveGate.guard`.  Swallows the block's exception, asks the
    group whether anybody has one, and re-raises in the matching form on every rank."""

    def __init__(self, gate: "CollectiveGate", what: str):
        self._gate, self._what = gate, what

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        anyone_failed = self._gate.agree_bool(exc is not None, op="any")
        if not anyone_failed:
            return False
        me = self._gate.rank
        if exc is None:
            raise PeerFailure(
                f"[{self._what}] succeeded on rank {me} but FAILED on at least one peer, so this rank stops here "
                "rather than entering the next collective alone. The failing rank's log holds the original "
                "traceback.")
        raise CollectiveFailure(
            f"[{self._what}] failed on rank {me} (surfaced collectively so no rank proceeds alone): "
            f"{type(exc).__name__}: {exc}") from exc


class CollectiveGate:
    """Group-wide agreement for one process group.  Every method is COLLECTIVE -- all ranks of the
    group call it, in the same order."""

    def __init__(self, group=None, device=None, timeout_s: float = DEFAULT_BARRIER_TIMEOUT_S):
        if not dist.is_available() or not dist.is_initialized():
            raise RuntimeError(
                "CollectiveGate needs an initialized torch.distributed process group; call "
                "init_process_group first. Constructing it earlier hides the real error behind a "
                "collective failure several frames later.")
        self.group = group
        self.timeout_s = timeout_s
        self.device = torch.device(device) if device is not None else self._vote_device(group)

    @staticmethod
    def _vote_device(group) -> torch.device:
        """Where the one-element vote tensor lives: the current GPU under NCCL, the host otherwise."""
        on_gpu = "nccl" in str(dist.get_backend(group)) and torch.cuda.is_available()
        return torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group)

    # -----------------------------------------------------------------------------------------
    def agree_bool(self, local: bool, *, op: str = "any") -> bool:
        """Reduce one boolean over the group: ``"any"`` is true when at least one rank said True,
        ``"all"`` only when every rank did."""
        reducers = {"any": dist.ReduceOp.MAX, "all": dist.ReduceOp.MIN}
        if op not in reducers:
            raise ValueError(f"op must be 'any' or 'all'; got {op!r}")
        vote = torch.full((1,), int(bool(local)), dtype=torch.int32, device=self.device)
        dist.all_reduce(vote, op=reducers[op], group=self.group)
        return int(vote.item()) == 1

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        """A barrier with a bound: :class:`BarrierTimeout` instead of an endless wait.

        ``CPO_BARRIER_WAIT`` picks the waiting style: ``poll`` (default) polls the asynchronous
        handle, ``wait`` blocks on it with a timeout, ``sync`` is the plain blocking barrier (no
        bound; for backends whose handles cannot be polled)."""
        bound_s = self.timeout_s if timeout_s is None else timeout_s
        if bound_s <= 0:
            raise ValueError(f"barrier timeout must be positive; got {bound_s}")
        style = os.environ.get("CPO_BARRIER_WAIT", "poll")
        if style == "sync":
            extra = {"device_ids": [self.device.index]} if self.device.type == "cuda" else {}
            dist.barrier(group=self.group, **extra)
            return
        handle = dist.barrier(group=self.group, async_op=True)
        if handle is None:  # a one-rank group has nothing to wait for
            return
        if not _ASYNC_WAITS.get(style, _wait_by_polling)(handle, bound_s):
            raise BarrierTimeout(
                f"rank {self.rank} waited {bound_s:.0f}s at a collective barrier and at least one peer never "
                "arrived. The group is now desynchronized -- do NOT enter another collective. A peer has died, "
                "hung, or taken a divergent path (a per-rank skip or an unguarded exception are the usual causes).")

    def guard(self, what: str) -> _GuardedRegion:
        """``with gate.guard("build"): ...`` -- if the block raises on ANY rank, EVERY rank raises after
        one reduction: :class:`CollectiveFailure` (chained to the cause) where it happened,
        :class:`PeerFailure` elsewhere.  A block that succeeds everywhere is left untouched."""
        return _GuardedRegion(self, what)

    def should_skip(self, local_reason: Optional[str]) -> Optional[str]:
        """All ranks skip or none does.  Returns ``None`` to carry on, otherwise the reason: this
        rank's own if it had one, a note that a peer asked if it did not."""
        if self.agree_bool(local_reason is not None, op="any"):
            return local_reason or "a peer rank requested a skip (this rank's own predicate passed)"
        return None
