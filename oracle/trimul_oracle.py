"""CPU oracle for the TriMul forward -- TEST INFRASTRUCTURE, not a compute path.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` may import this module, and only as the checker (or as the timed CPU baseline); the
product package never does.

It restates, op for op in fp32 on the CPU, the reference's eager TriMul
(``fold_cp_ops/workflows/trimul_autotune.py:1505-1525``, ``trimul_ref``):

     1  xn    = LayerNorm(x; gamma_in, beta_in, eps)
     2  p_in  = xn @ p_in_w^T + p_in_b            (2D wide)
     3  g_in  = xn @ g_in_w^T + g_in_b
     4  ab    = p_in * sigmoid(g_in)
     5  ab    = ab * mask[..., None]               (mask reaches a|b only, never the output gate)
     6  a, b  = ab[..., :D], ab[..., D:]
     7  tri   = einsum('bikd,bjkd->bijd', a, b)    outgoing
              = einsum('bkid,bkjd->bijd', a, b)    incoming
     8  trin  = LayerNorm(tri; gamma_out, beta_out, eps)
     9  p_out = trin @ p_out_w^T + p_out_b
    10  g_out = xn @ g_out_w^T + g_out_b           (reads xn, the FRONT LayerNorm, not trin)
    11-12  out = p_out * sigmoid(g_out)

The LayerNorm is written out (mean / biased variance) instead of calling
``torch.nn.functional.layer_norm`` so that the restatement is independent of the call the
reference makes.  Pinned against the reference itself: ``tests/golden/`` holds outputs of the
reference's ``trimul_ref`` on seeded inputs (made by ``tests/golden/make_golden.py``), and
``tests/test_oracle.py`` checks this file against them and, when the reference checkout is
importable, against ``trimul_ref`` directly.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

W_KEYS = ("norm_in_w", "norm_in_b", "p_in_w", "g_in_w", "norm_out_w", "norm_out_b", "p_out_w", "g_out_w")
W_PROJ_BIAS_KEYS = ("p_in_b", "g_in_b", "p_out_b", "g_out_b")


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """LayerNorm over the last axis with biased variance (what F.layer_norm computes)."""
    x = x.float()
    mean = x.mean(dim=-1, keepdim=True)
    xc = x - mean
    var = (xc * xc).mean(dim=-1, keepdim=True)
    y = xc * torch.rsqrt(var + eps) * w.float()
    return y if b is None else y + b.float()


def _f(t):
    return None if t is None else t.float()


def trimul_stages(x, direction, mask, norm_in_w, norm_in_b, p_in_w, g_in_w, norm_out_w, norm_out_b, p_out_w,
                  g_out_w, p_in_b=None, g_in_b=None, p_out_b=None, g_out_b=None, eps=1e-5,
                  round_bf16: bool = False) -> Dict[str, torch.Tensor]:
    """Every intermediate of the forward in fp32.

    ``round_bf16=True`` additionally rounds to bf16 at the points where the fused kernel chain
    stores bf16 (the LayerNorm outputs feeding the tensor core, a|b, the output gate, tri), which
    gives per-kernel tests a tight target; the parity bar itself is always the unrounded oracle.
    """
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}")
    rnd = (lambda t: t.to(torch.bfloat16).float()) if round_bf16 else (lambda t: t)
    D = x.shape[-1]
    xn = rnd(layer_norm(x, norm_in_w, norm_in_b, eps))
    p_in = xn @ p_in_w.float().T
    g_in = xn @ g_in_w.float().T
    if p_in_b is not None:
        p_in = p_in + p_in_b.float()
    if g_in_b is not None:
        g_in = g_in + g_in_b.float()
    ab = p_in * torch.sigmoid(g_in)
    if mask is not None:
        ab = ab * mask.float().unsqueeze(-1)
    ab = rnd(ab)
    a, b = ab[..., :D], ab[..., D:]
    if direction == "outgoing":
        tri = torch.einsum("bikd,bjkd->bijd", a, b)
    else:
        tri = torch.einsum("bkid,bkjd->bijd", a, b)
    tri = rnd(tri)
    trin = rnd(layer_norm(tri, norm_out_w, norm_out_b, eps))
    p_out = trin @ p_out_w.float().T
    if p_out_b is not None:
        p_out = p_out + p_out_b.float()
    g_out = xn @ g_out_w.float().T
    if g_out_b is not None:
        g_out = g_out + g_out_b.float()
    gate = rnd(torch.sigmoid(g_out))
    out = p_out * gate
    return {"xn": xn, "a": a, "b": b, "tri": tri, "trin": trin, "gate": gate, "out": out}


def trimul_eager_module(x, direction, mask=None, *, eps=1e-5, **w) -> torch.Tensor:
    """The same forward in the spelling of the reference's eager ``nn.Module``
    (``benchmark/distributed/trimul_dtensor_reference.py:1841-1847``: ``nn.LayerNorm`` / ``nn.Linear``
    submodules, the mask applied before the chunk, one ``einsum`` at fp32, the output gate on ``xn``),
    written with the functional forms of those modules.  Equal to :func:`trimul_oracle` up to fp32
    summation order; on a CPU it is the faster of the two spellings (fused LayerNorm, biases folded into
    the GEMMs), which is why the timed CPU baseline reports both."""
    import torch.nn.functional as F

    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}")
    D = x.shape[-1]
    x = x.float()
    xn = F.layer_norm(x, (D,), _f(w["norm_in_w"]), _f(w.get("norm_in_b")), eps)
    ab = F.linear(xn, _f(w["p_in_w"]), _f(w.get("p_in_b"))) * torch.sigmoid(F.linear(xn, _f(w["g_in_w"]), _f(w.get("g_in_b"))))
    if mask is not None:
        ab = ab * mask.float().unsqueeze(-1)
    a, b = torch.chunk(ab, 2, dim=-1)
    tri = torch.einsum("bikd,bjkd->bijd" if direction == "outgoing" else "bkid,bkjd->bijd", a, b)
    trin = F.layer_norm(tri, (D,), _f(w["norm_out_w"]), _f(w.get("norm_out_b")), eps)
    return F.linear(trin, _f(w["p_out_w"]), _f(w.get("p_out_b"))) * torch.sigmoid(F.linear(xn, _f(w["g_out_w"]), _f(w.get("g_out_b"))))


def trimul_oracle_tiled(x, direction, mask=None, *, row_tile: int = 512, on_tile=None, eps=1e-5, **w):
    """The oracle evaluated one ``(row_tile x row_tile)`` block of the OUTPUT grid at a time, the contraction
    index kept whole -- the job of the reference's ``trimul_ref_chunked``
    (``fold_cp_ops/workflows/trimul_autotune.py:1727-1815``): peak memory is O(row_tile * N * D) instead of
    O(N^2 * D), so a large-N output can be checked without ever holding the fp32 oracle.

    Without ``on_tile`` the blocks are assembled and returned (equal to :func:`trimul_oracle` up to fp32
    summation order).  With ``on_tile(i0, i1, j0, j1, block)`` every fp32 block ``(B, i1-i0, j1-j0, D)`` is
    handed to the callback instead and ``None`` is returned.  ``row_tile`` need not divide N."""
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"direction must be 'outgoing' or 'incoming'; got {direction!r}")
    B, N, _, D = x.shape
    T = int(row_tile) if row_tile and int(row_tile) > 0 else N
    outgoing = direction == "outgoing"

    def half(lo, hi, which):
        # gated projection of the input lines [lo, hi) (rows for outgoing, columns for incoming), a or b half
        xs = x[:, lo:hi] if outgoing else x[:, :, lo:hi]
        xn = layer_norm(xs, w["norm_in_w"], w.get("norm_in_b"), eps)
        p = xn @ w["p_in_w"].float().T
        g = xn @ w["g_in_w"].float().T
        if w.get("p_in_b") is not None:
            p = p + w["p_in_b"].float()
        if w.get("g_in_b") is not None:
            g = g + w["g_in_b"].float()
        ab = p * torch.sigmoid(g)
        if mask is not None:
            ms = mask[:, lo:hi] if outgoing else mask[:, :, lo:hi]
            ab = ab * ms.float().unsqueeze(-1)
        return ab[..., :D] if which == 0 else ab[..., D:]

    out = None if on_tile is not None else torch.empty((B, N, N, D), dtype=torch.float32, device=x.device)
    for i0 in range(0, N, T):
        i1 = min(i0 + T, N)
        a = half(i0, i1, 0)
        for j0 in range(0, N, T):
            j1 = min(j0 + T, N)
            b = half(j0, j1, 1)
            tri = torch.einsum("bikd,bjkd->bijd" if outgoing else "bkid,bkjd->bijd", a, b)
            p_out = layer_norm(tri, w["norm_out_w"], w.get("norm_out_b"), eps) @ w["p_out_w"].float().T
            if w.get("p_out_b") is not None:
                p_out = p_out + w["p_out_b"].float()
            g_out = layer_norm(x[:, i0:i1, j0:j1], w["norm_in_w"], w.get("norm_in_b"), eps) @ w["g_out_w"].float().T
            if w.get("g_out_b") is not None:
                g_out = g_out + w["g_out_b"].float()
            block = p_out * torch.sigmoid(g_out)
            if on_tile is not None:
                on_tile(i0, i1, j0, j1, block)
            else:
                out[:, i0:i1, j0:j1] = block
    return out


def trimul_oracle(x, direction, mask=None, *, eps=1e-5, **w) -> torch.Tensor:
    """``(B, N, N, D)`` fp32 TriMul forward; keyword weights as in the reference's 12-key dict."""
    return trimul_stages(x, direction, mask, eps=eps, **w)["out"]


# -------------------------------------------------------------------------------------------------
# seeded synthetic inputs (numpy's frozen RandomState stream => identical on every machine)
# -------------------------------------------------------------------------------------------------
def make_case(B: int, N: int, D: int, seed: int, *, ln_affine: bool = True, bias: str = "all",
              mask: str = "none", w_std: Optional[float] = None, bias_std: float = 0.02,
              ln_bias_std: float = 0.1) -> Dict[str, Optional[torch.Tensor]]:
    """Synthetic TriMul inputs with the value distributions the benchmark configurations name.

    x ~ N(0,1); LayerNorm gain 1 + 0.1 N(0,1), bias ``ln_bias_std`` N(0,1) (identity when
    ``ln_affine`` is False); the six projection matrices ~ N(0, 1/D); projection biases
    ``bias_std`` N(0,1) for ``bias`` in {"all", "out"(p_out/g_out only), "none"}; ``mask`` in
    {"none", "ones", "pad" (outer product of a token mask whose last 10% is zero), "random"}.
    Everything is returned as fp32 CPU tensors; callers round to bf16 where the kernels need it.
    """
    rs = np.random.RandomState(seed)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    std = (1.0 / np.sqrt(D)) if w_std is None else w_std
    case: Dict[str, Optional[torch.Tensor]] = {}
    case["x"] = t(rs.standard_normal((B, N, N, D)))
    for nm in ("norm_in", "norm_out"):
        if ln_affine:
            case[nm + "_w"] = t(1.0 + 0.1 * rs.standard_normal(D))
            case[nm + "_b"] = t(ln_bias_std * rs.standard_normal(D))
        else:
            case[nm + "_w"] = torch.ones(D)
            case[nm + "_b"] = torch.zeros(D)
    case["p_in_w"] = t(std * rs.standard_normal((2 * D, D)))
    case["g_in_w"] = t(std * rs.standard_normal((2 * D, D)))
    case["p_out_w"] = t(std * rs.standard_normal((D, D)))
    case["g_out_w"] = t(std * rs.standard_normal((D, D)))
    pb = {"p_in_b": 2 * D, "g_in_b": 2 * D, "p_out_b": D, "g_out_b": D}
    for k, n in pb.items():
        v = t(bias_std * rs.standard_normal(n))  # always drawn so the stream does not depend on `bias`
        keep = bias == "all" or (bias == "out" and k in ("p_out_b", "g_out_b"))
        case[k] = v if keep else None
    if mask == "none":
        case["mask"] = None
    elif mask == "ones":
        case["mask"] = torch.ones(B, N, N)
    elif mask == "pad":
        tok = torch.ones(N)
        tok[N - max(1, N // 10):] = 0.0
        case["mask"] = (tok[:, None] * tok[None, :]).expand(B, N, N).contiguous()
    elif mask == "random":
        case["mask"] = t((rs.uniform(size=(B, N, N)) > 0.3).astype(np.float32))
    else:
        raise ValueError(f"unknown mask kind {mask!r}")
    return case


def weights_of(case: Dict[str, Optional[torch.Tensor]]) -> Dict[str, Optional[torch.Tensor]]:
    return {k: case[k] for k in W_KEYS + W_PROJ_BIAS_KEYS}


def bf16_round_case(case: Dict[str, Optional[torch.Tensor]]) -> Dict[str, Optional[torch.Tensor]]:
    """What the kernels actually receive: x and the six projection matrices rounded to bf16 (kept
    as fp32 values); LayerNorm parameters and biases stay fp32 (the reference refuses non-fp32
    LayerNorm parameters: fold_cp_ops/distributed/workflows/trimul_autotuned.py:4263-4274)."""
    out = dict(case)
    for k in ("x", "p_in_w", "g_in_w", "p_out_w", "g_out_w"):
        out[k] = case[k].to(torch.bfloat16).float()
    return out


def tolerance_bound(ref: torch.Tensor, atol: float = 2e-2, rtol: float = 6e-2) -> torch.Tensor:
    """Per-element bound of the reference's distributed parity gate
    (tests/distributed/workflows/test_trimul_autotuned.py:556): |err| <= atol + rtol * |ref|."""
    return atol + rtol * ref.abs()


def cp1_bound(ref: torch.Tensor) -> torch.Tensor:
    """Per-element bound of the reference's cp=1 workflow gate
    (tests/workflows/test_trimul_autotune.py:78-92): 0.01 * max|ref| + 0.01 * |ref|."""
    return 0.01 * ref.abs().max() + 0.01 * ref.abs()
