"""Single-GPU fused TriMul: ``trimul_autotuned``.

Drop-in for the reference's cp=1 front door ``fold_cp_ops/workflows/trimul_autotune.py:1531``
(same name, argument order and validation sentences).  The reference picks one of five SM90
kernel chains ("combos") by heuristic or autotune; this build has exactly one chain -- the three
sm_100a kernels -- so ``select`` is validated and otherwise ignored.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch
from torch import Tensor

from ..engine import TriMulEngine

__all__ = ["trimul_autotuned", "TRIMUL_VARIANTS", "clear_cache"]

#: the kernel chains this build can run (the reference lists five SM90 combos here)
TRIMUL_VARIANTS = ("sm100_fused",)

#: engines (packed weights + workspaces) keyed on the identity of the twelve weight tensors.  An entry
#: keeps references to those tensors, so their storage cannot be freed and handed to another model of the
#: same shapes while the entry lives.  The key includes each tensor's version counter: in-place updates
#: through autograd-visible ops (``copy_``, ``add_`` ...) repack the weights; writes that bypass the
#: counter (``param.data.copy_(...)``) do NOT -- call :func:`clear_cache` after loading weights that way.
_ENGINE_CACHE: "OrderedDict[tuple, tuple]" = OrderedDict()
_ENGINE_CACHE_CAP = 8


def _weight_key(t: Optional[Tensor]):
    if t is None:
        return None
    return (t.data_ptr(), t._version, tuple(t.shape), t.dtype, str(t.device))


def _engine_for(device, eps, w: dict) -> TriMulEngine:
    key = (str(device), float(eps)) + tuple(_weight_key(w[k]) for k in sorted(w))
    entry = _ENGINE_CACHE.get(key)
    if entry is None:
        entry = (TriMulEngine(w, device=device, eps=eps), tuple(w[k] for k in sorted(w)))
        _ENGINE_CACHE[key] = entry
        while len(_ENGINE_CACHE) > _ENGINE_CACHE_CAP:
            _ENGINE_CACHE.popitem(last=False)[1][0].free()
    else:
        _ENGINE_CACHE.move_to_end(key)
    return entry[0]


def clear_cache() -> None:
    """Drop every cached single-GPU engine (packed weights, workspaces).  Needed after weights were
    overwritten in a way their version counters do not see."""
    while _ENGINE_CACHE:
        _ENGINE_CACHE.popitem()[1][0].free()


def engines_for_weights(w: dict):
    """The cached engines that were built from exactly these weight tensors (by identity)."""
    mine = {id(t) for t in w.values() if t is not None}
    return [eng for eng, kept in _ENGINE_CACHE.values() if {id(t) for t in kept if t is not None} <= mine and mine]


def trimul_autotuned(
    x: Tensor,
    norm_in_w: Tensor,
    norm_in_b: Optional[Tensor] = None,
    p_in_w: Tensor = None,
    g_in_w: Tensor = None,
    norm_out_w: Tensor = None,
    norm_out_b: Optional[Tensor] = None,
    p_out_w: Tensor = None,
    g_out_w: Tensor = None,
    p_in_b: Optional[Tensor] = None,
    g_in_b: Optional[Tensor] = None,
    p_out_b: Optional[Tensor] = None,
    g_out_b: Optional[Tensor] = None,
    mask: Optional[Tensor] = None,
    direction: str = "outgoing",
    eps: float = 1e-5,
    out: Optional[Tensor] = None,
    select: str = "heuristic",
    _config=None,
) -> Tensor:
    """``(B, N, N, D)`` -> ``(B, N, N, D)`` in ``x.dtype``; bf16 tensor-core compute, fp32 statistics.

    Raises ``ValueError`` for an unknown ``direction`` / ``select``, a non-square token grid,
    ``N % 8 != 0``, ``D % 8 != 0`` (or a width the kernels do not cover), non-fp32 LayerNorm
    gains, and mis-shaped projection matrices or mask.
    """
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}")
    if select not in ("heuristic", "autotune", "default"):
        raise ValueError(f"select must be 'heuristic', 'autotune' or 'default'; got {select!r}")
    if x.dim() != 4:
        raise ValueError(f"x must be (B, N, N, D); got {tuple(x.shape)}")
    B, N, N2, D = x.shape
    if N != N2:
        raise ValueError(f"x must be (B, N, N, D) with a square token axis; got {N} x {N2}")
    if N % 8 != 0:
        raise ValueError(
            f"N must be 16-byte aligned (N % 8 == 0 for a 16-bit activation); got N={N}. The "
            f"token-pair einsum contracts (N, N) operands, so N is their row pitch, and NO combo "
            f"can run a shape that breaks it.")
    if D % 8 != 0:
        raise ValueError(f"D must be 16-byte aligned (D % 8 == 0 for a 16-bit activation); got D={D}.")
    if norm_in_w.dim() != 1 or norm_in_w.dtype != torch.float32:
        raise ValueError(f"norm_in_w must be a ({D},) float32 tensor; got {tuple(norm_in_w.shape)}")
    if norm_out_w.dim() != 1 or norm_out_w.dtype != torch.float32:
        raise ValueError(f"norm_out_w must be a ({D},) float32 tensor; got {tuple(norm_out_w.shape)}")
    if tuple(p_in_w.shape) != (2 * D, D) or tuple(g_in_w.shape) != (2 * D, D):
        raise ValueError(f"p_in_w and g_in_w must both be (2D, D) = ({2 * D}, {D}); got "
                         f"{tuple(p_in_w.shape)} and {tuple(g_in_w.shape)}")
    if tuple(p_out_w.shape) != (D, D) or tuple(g_out_w.shape) != (D, D):
        raise ValueError(f"p_out_w and g_out_w must both be (D, D) = ({D}, {D}); got "
                         f"{tuple(p_out_w.shape)} and {tuple(g_out_w.shape)}")
    if mask is not None and tuple(mask.shape[-2:]) != (N, N):
        raise ValueError(f"mask must be (..., N, N) = (..., {N}, {N}); got {tuple(mask.shape)}")
    if not x.is_cuda:
        raise RuntimeError("trimul_autotuned needs a CUDA tensor: the sm_100a kernels are the only code path")

    w = dict(norm_in_w=norm_in_w, norm_in_b=norm_in_b, p_in_w=p_in_w, g_in_w=g_in_w, norm_out_w=norm_out_w,
             norm_out_b=norm_out_b, p_out_w=p_out_w, g_out_w=g_out_w, p_in_b=p_in_b, g_in_b=g_in_b,
             p_out_b=p_out_b, g_out_b=g_out_b)
    eng = _engine_for(x.device, eps, w)
    res = eng.forward(x, direction, None if mask is None else mask.reshape(B, N, N))
    if res.dtype is not x.dtype:
        res = res.to(x.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res
