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

#: submodule -> (kind, output width as a multiple of D).  Everything below is derived from this table.
_SUBMODULES = {"norm_in": ("norm", 1), "p_in": ("linear", 2), "g_in": ("linear", 2),
               "norm_out": ("norm", 1), "p_out": ("linear", 1), "g_out": ("linear", 1)}


def _required_slots():
    """(submodule, attribute, w-key) of the eight tensors every layer has, in ``W_KEYS`` order."""
    slots = {}
    for sub, (kind, _) in _SUBMODULES.items():
        slots[f"{sub}_w"] = (sub, "weight")
        if kind == "norm":
            slots[f"{sub}_b"] = (sub, "bias")
    return [(*slots[key], key) for key in W_KEYS]


def _bias_slots():
    return [(key[:-2], key) for key in W_PROJ_BIAS_KEYS]


def weights_from_trimul_module(module: torch.nn.Module, *, dtype: Optional[torch.dtype] = None, device=None,
                               detach: bool = True) -> dict:
    """Read the 12-key dict off any module exposing ``norm_in/p_in/g_in/norm_out/p_out/g_out``.

    Raises ``AttributeError`` naming the missing submodule or parameter."""

    def convert(t):
        t = t.detach() if detach else t
        t = t if dtype is None else t.to(dtype)
        return t if device is None else t.to(device)

    missing = [sub for sub in _SUBMODULES if getattr(module, sub, None) is None]
    if missing:
        raise AttributeError(f"module {type(module).__name__} has no submodule '{missing[0]}'; "
                             "weights_from_trimul_module expects a TriangularMultiplication layer "
                             "(norm_in/p_in/g_in/norm_out/p_out/g_out).")
    out: dict = {}
    for sub, attr, key in _required_slots():
        tensor = getattr(getattr(module, sub), attr, None)
        if tensor is None:
            raise AttributeError(f"submodule '{sub}' has no '{attr}' (expected for w-key '{key}').")
        out[key] = convert(tensor)
    for sub, key in _bias_slots():
        bias = getattr(getattr(module, sub), "bias", None)
        out[key] = bias if bias is None else convert(bias)
    return out


def trimul_module_from_weights(w: dict, *, dtype: Optional[torch.dtype] = None) -> torch.nn.Module:
    """Inverse adapter: a bare module with the six submodules, sharing storage with ``w``.

    Raises ``KeyError`` if a ``W_KEYS`` entry is absent, ``ValueError`` if one is ``None``."""
    absent = [key for key in W_KEYS if key not in w]
    if absent:
        raise KeyError(f"trimul_module_from_weights: weight dict is missing '{absent[0]}'")
    empty = [key for key in W_KEYS if w[key] is None]
    if empty:
        raise ValueError(f"trimul_module_from_weights: '{empty[0]}' is None; every one of W_KEYS must be a tensor.")

    def frozen(t):
        return torch.nn.Parameter(t if dtype is None else t.to(dtype), requires_grad=False)

    width = int(w["norm_in_w"].shape[-1])
    has_bias = {sub: w.get(key) is not None for sub, key in _bias_slots()}
    layer = torch.nn.Module()
    for sub, (kind, mult) in _SUBMODULES.items():
        built = (torch.nn.LayerNorm(width, eps=1e-5) if kind == "norm"
                 else torch.nn.Linear(width, mult * width, bias=has_bias[sub]))
        layer.add_module(sub, built)
    with torch.no_grad():
        for sub, attr, key in _required_slots():
            setattr(getattr(layer, sub), attr, frozen(w[key]))
        for sub, key in _bias_slots():
            if has_bias[sub]:
                getattr(layer, sub).bias = frozen(w[key])
    return layer.eval()
