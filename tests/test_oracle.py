"""The CPU oracle is pinned against the reference: golden vectors made by the reference's own
``trimul_ref`` (tests/golden/make_golden.py) and, when the reference checkout is importable, the
reference called directly."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle.trimul_oracle import (bf16_round_case, cp1_bound, make_case, tolerance_bound, trimul_oracle,
                                  trimul_stages, weights_of)
from tests.golden.make_golden import CASES, input_digest

from tests.conftest import reference_root

REFERENCE_ROOT = str(reference_root() or "")


def _case(name):
    kw = dict(CASES[name])
    direction = kw.pop("direction")
    return bf16_round_case(make_case(**kw)), direction


@pytest.mark.parametrize("name", sorted(CASES))
def test_inputs_are_reproducible(name, golden):
    case, _ = _case(name)
    want = bytes(golden[name + "__digest"].tobytes()).hex()
    assert input_digest(case) == want, "seeded inputs differ from the ones the golden vectors were made with"


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_golden(name, golden):
    case, direction = _case(name)
    got = trimul_oracle(case["x"], direction, case["mask"], eps=1e-5, **weights_of(case))
    ref = torch.from_numpy(golden[name])
    assert got.shape == ref.shape and got.dtype == torch.float32
    # both are fp32 evaluations of the same twelve ops; only summation order may differ
    err = (got - ref).abs()
    assert err.max().item() <= 2e-5 * max(1.0, ref.abs().max().item()), err.max().item()


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_oracle_matches_reference_eager_module_golden(direction, golden):
    case = bf16_round_case(make_case(B=1, N=16, D=128, seed=107, ln_affine=True, bias="none", mask="random"))
    got = trimul_oracle(case["x"], direction, case["mask"], eps=1e-5, **weights_of(case))
    ref = torch.from_numpy(golden[f"eager_{direction}_n16_d128"])
    assert (got - ref).abs().max().item() <= 2e-5 * max(1.0, ref.abs().max().item())


_LIVE_SNIPPET = """
import sys, numpy as np, torch
sys.dont_write_bytecode = True
sys.path.insert(0, {repo!r}); sys.path.insert(0, {ref!r})   # the reference's own package wins the name
from fold_cp_ops.workflows.trimul_autotune import trimul_ref, trimul_ref_chunked
from oracle.trimul_oracle import bf16_round_case, make_case, weights_of
out = {{}}
for direction in ("outgoing", "incoming"):
    for bias, mask in (("none", "none"), ("all", "random"), ("out", "pad")):
        case = bf16_round_case(make_case(B=2, N=24, D=128, seed=7, bias=bias, mask=mask))
        out[f"{{direction}}_{{bias}}_{{mask}}"] = trimul_ref(case["x"], direction, case["mask"], **weights_of(case), eps=1e-5).numpy()
    case = bf16_round_case(make_case(B=1, N=40, D=128, seed=9, bias="all", mask="random"))
    out[f"chunked_{{direction}}"] = trimul_ref_chunked(case["x"], direction, case["mask"], **weights_of(case), eps=1e-5, row_tile=16).numpy()
np.savez({dst!r}, **out)
"""


@pytest.fixture(scope="module")
def live_reference(tmp_path_factory):
    """Outputs of the reference's own trimul_ref, computed in a child process whose import path
    puts the reference checkout first (this repository ships an alias package of the same name)."""
    if not os.path.isdir(os.path.join(REFERENCE_ROOT, "fold_cp_ops")):
        pytest.skip("reference checkout not present")
    import subprocess

    dst = str(tmp_path_factory.mktemp("live") / "ref.npz")
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = _LIVE_SNIPPET.format(repo=repo, ref=REFERENCE_ROOT, dst=dst)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    if proc.returncode != 0:
        pytest.skip(f"reference not importable here: {proc.stderr[-400:]}")
    return np.load(dst)


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
@pytest.mark.parametrize("bias,mask", [("none", "none"), ("all", "random"), ("out", "pad")])
def test_oracle_matches_live_reference(direction, bias, mask, live_reference):
    case = bf16_round_case(make_case(B=2, N=24, D=128, seed=7, bias=bias, mask=mask))
    ref = torch.from_numpy(live_reference[f"{direction}_{bias}_{mask}"])
    got = trimul_oracle(case["x"], direction, case["mask"], eps=1e-5, **weights_of(case))
    assert (got - ref).abs().max().item() <= 2e-5 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_tiled_oracle_matches_live_reference_chunked(direction, live_reference):
    from oracle.trimul_oracle import trimul_oracle_tiled

    case = bf16_round_case(make_case(B=1, N=40, D=128, seed=9, bias="all", mask="random"))
    ref = torch.from_numpy(live_reference[f"chunked_{direction}"])
    got = trimul_oracle_tiled(case["x"], direction, case["mask"], row_tile=16, eps=1e-5, **weights_of(case))
    assert (got - ref).abs().max().item() <= 2e-5 * max(1.0, ref.abs().max().item())


def test_mask_reaches_dual_only_and_gate_reads_xn():
    """Semantics pins of the reference (tests/workflows/test_trimul_autotune.py:648-667): a zero mask
    zeroes tri (so out = gate * (beta_out . W + b)), and the gate does not depend on the mask."""
    case = bf16_round_case(make_case(B=1, N=8, D=128, seed=3, bias="all", mask="ones"))
    w = weights_of(case)
    full = trimul_stages(case["x"], "outgoing", case["mask"], **w)
    zero = trimul_stages(case["x"], "outgoing", torch.zeros_like(case["mask"]), **w)
    assert torch.equal(full["gate"], zero["gate"])
    assert zero["tri"].abs().max().item() == 0.0
    assert zero["a"].abs().max().item() == 0.0


def test_directions_differ_and_transpose_relation():
    """tri_incoming(x) == tri_outgoing(x^T): transposing the pair tensor in (i, j) swaps the index
    the contraction runs over (the output gate stays at its own (i, j), so only tri relates)."""
    case = bf16_round_case(make_case(B=1, N=8, D=128, seed=5, bias="all", mask="random"))
    w = weights_of(case)
    inc = trimul_stages(case["x"], "incoming", case["mask"], **w)
    out_t = trimul_stages(case["x"].transpose(1, 2).contiguous(), "outgoing",
                          case["mask"].transpose(1, 2).contiguous(), **w)
    assert (inc["tri"] - out_t["tri"]).abs().max().item() < 1e-4
    out = trimul_stages(case["x"], "outgoing", case["mask"], **w)
    assert (inc["out"] - out["out"]).abs().max().item() > 1e-2


def test_bad_direction_raises():
    case = make_case(B=1, N=8, D=128, seed=1)
    with pytest.raises(ValueError):
        trimul_oracle(case["x"], "sideways", None, **weights_of(case))


def test_bounds_shapes():
    ref = torch.randn(4, 4)
    assert tolerance_bound(ref).shape == ref.shape
    assert cp1_bound(ref).shape == ref.shape


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_eager_module_spelling_equals_the_restatement(direction):
    """The timed CPU baseline may use the eager-module spelling (fused LayerNorm, biases inside the
    GEMMs): it must be the same function as the op-for-op restatement, up to fp32 summation order."""
    from oracle.trimul_oracle import make_case, trimul_eager_module, trimul_oracle, weights_of

    case = make_case(2, 40, 128, seed=31, bias="all", mask="pad")
    a = trimul_oracle(case["x"], direction, case["mask"], **weights_of(case))
    b = trimul_eager_module(case["x"], direction, case["mask"], **weights_of(case))
    assert (a - b).abs().max().item() <= 2e-4 * max(1.0, a.abs().max().item())
    nomask = trimul_eager_module(case["x"], direction, None, **weights_of(case))
    assert torch.allclose(nomask, trimul_oracle(case["x"], direction, None, **weights_of(case)), atol=2e-4, rtol=1e-4)


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_tiled_oracle_equals_the_full_oracle(direction):
    """The memory-frugal form (output grid in blocks, contraction whole; the reference's ``trimul_ref_chunked``)
    is the same function, with a block size that does not divide N, and streams the same blocks."""
    from oracle.trimul_oracle import make_case, trimul_oracle, trimul_oracle_tiled, weights_of

    case = make_case(2, 40, 128, seed=33, bias="all", mask="random")
    full = trimul_oracle(case["x"], direction, case["mask"], **weights_of(case))
    tiled = trimul_oracle_tiled(case["x"], direction, case["mask"], row_tile=16, **weights_of(case))
    assert (tiled - full).abs().max().item() <= 2e-5 * max(1.0, full.abs().max().item())
    seen = torch.zeros(40, 40, dtype=torch.int32)
    worst = [0.0]

    def on_tile(i0, i1, j0, j1, block):
        seen[i0:i1, j0:j1] += 1
        worst[0] = max(worst[0], (block - full[:, i0:i1, j0:j1]).abs().max().item())

    assert trimul_oracle_tiled(case["x"], direction, case["mask"], row_tile=16, on_tile=on_tile, **weights_of(case)) is None
    assert bool((seen == 1).all()) and worst[0] <= 2e-5 * max(1.0, full.abs().max().item())
