"""nn.Module <-> 12-key weight dict adapters for the fused TriMul.

Mirrors ``fold_cp_ops/distributed/trimul_weights.py:70-262``.  ``nn.Linear.weight`` is (out, in)
and applied as ``x @ W^T``; rows ``[0:D]`` of ``p_in_w`` / ``g_in_w`` are the **a** half, rows
``[D:2D]`` the **b** half.  Unlike the reference (whose front store could not fuse them), the
input-projection biases ``p_in_b`` / ``g_in_b`` are carried: the sm_100a projection kernel adds
all four projection biases in its epilogue.
"""
from __future__ import annotations

from typing import Optional

import torch

#: the eight weights every layer has
W_KEYS = ("norm_in_w", "norm_in_b", "p_in_w", "g_in_w", "norm_out_w", "norm_out_b", "p_out_w", "g_out_w")
#: the four optional projection biases (``None`` when the Linear has none)
W_PROJ_BIAS_KEYS = ("p_in_b", "g_in_b", "p_out_b", "g_out_b")

_PARAMS = (("norm_in", "weight", "norm_in_w"), ("norm_in", "bias", "norm_in_b"), ("p_in", "weight", "p_in_w"),
           ("g_in", "weight", "g_in_w"), ("norm_out", "weight", "norm_out_w"), ("norm_out", "bias", "norm_out_b"),
           ("p_out", "weight", "p_out_w"), ("g_out", "weight", "g_out_w"))
_BIASES = (("p_in", "p_in_b"), ("g_in", "g_in_b"), ("p_out", "p_out_b"), ("g_out", "g_out_b"))


def _prep(t, dtype, device, detach):
    if detach:
        t = t.detach()
    if dtype is not None:
        t = t.to(dtype)
    if device is not None:
        t = t.to(device)
    return t


def weights_from_trimul_module(module: torch.nn.Module, *, dtype: Optional[torch.dtype] = None, device=None,
                               detach: bool = True) -> dict:
    """Read the 12-key dict off any module exposing ``norm_in/p_in/g_in/norm_out/p_out/g_out``.

    Raises ``AttributeError`` naming the missing submodule or parameter."""
    w: dict = {}
    for sub, attr, key in _PARAMS:
        submod = getattr(module, sub, None)
        if submod is None:
            raise AttributeError(f"module {type(module).__name__} has no submodule '{sub}'; "
                                 "weights_from_trimul_module expects a TriangularMultiplication layer "
                                 "(norm_in/p_in/g_in/norm_out/p_out/g_out).")
        t = getattr(submod, attr, None)
        if t is None:
            raise AttributeError(f"submodule '{sub}' has no '{attr}' (expected for w-key '{key}').")
        w[key] = _prep(t, dtype, device, detach)
    for sub, key in _BIASES:
        b = getattr(getattr(module, sub), "bias", None)
        w[key] = None if b is None else _prep(b, dtype, device, detach)
    return w


def trimul_module_from_weights(w: dict, *, dtype: Optional[torch.dtype] = None) -> torch.nn.Module:
    """Inverse adapter: a bare module with the six submodules, sharing storage with ``w``.

    Raises ``KeyError`` if a ``W_KEYS`` entry is absent, ``ValueError`` if one is ``None``."""
    for key in W_KEYS:
        if key not in w:
            raise KeyError(f"trimul_module_from_weights: weight dict is missing '{key}'")
        if w[key] is None:
            raise ValueError(f"trimul_module_from_weights: '{key}' is None; every one of W_KEYS must be a tensor.")
    cast = (lambda t: t.to(dtype)) if dtype is not None else (lambda t: t)
    D = int(w["norm_in_w"].shape[-1])
    m = torch.nn.Module()
    m.norm_in = torch.nn.LayerNorm(D, eps=1e-5)
    m.norm_out = torch.nn.LayerNorm(D)
    m.p_in = torch.nn.Linear(D, 2 * D, bias=w.get("p_in_b") is not None)
    m.g_in = torch.nn.Linear(D, 2 * D, bias=w.get("g_in_b") is not None)
    m.p_out = torch.nn.Linear(D, D, bias=w.get("p_out_b") is not None)
    m.g_out = torch.nn.Linear(D, D, bias=w.get("g_out_b") is not None)
    param = lambda t: torch.nn.Parameter(cast(t), requires_grad=False)
    with torch.no_grad():
        for sub, attr, key in _PARAMS:
            setattr(getattr(m, sub), attr, param(w[key]))
        for sub, key in _BIASES:
            if w.get(key) is not None:
                getattr(m, sub).bias = param(w[key])
    return m.eval()
