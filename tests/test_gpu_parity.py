"""Parity of the sm_100a TriMul path against the CPU oracle -- every test calls through the C ABI.

Tolerances (bf16 storage at four points of the chain, fp32 accumulation and statistics):
  * whole forward vs the fp32 oracle: the reference's cp=1 gate ``0.01*max|ref| + 0.01*|ref|``
    per element (tests/workflows/test_trimul_autotune.py:78-92 of the reference) AND its
    distributed gate ``2e-2 + 6e-2*|ref|`` (tests/distributed/workflows/test_trimul_autotuned.py:556);
  * single kernels vs the oracle with bf16 rounding applied at the same points: a few bf16 ulps.
"""
import numpy as np
import pytest
import torch

from oracle.trimul_oracle import (bf16_round_case, cp1_bound, layer_norm, make_case, tolerance_bound, trimul_oracle,
                                  trimul_stages, weights_of)
from tests.golden.make_golden import CASES

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _engine(case, eps=1e-5):
    from fold_cp_ops_b200.engine import TriMulEngine

    return TriMulEngine(weights_of(case), device=torch.device(DEV), eps=eps)


def _run(case, direction, *, x_dtype=torch.bfloat16, mask_dtype=torch.float32):
    eng = _engine(case)
    x = case["x"].to(DEV).to(x_dtype)
    m = None if case["mask"] is None else case["mask"].to(DEV).to(mask_dtype)
    out = eng.forward(x, direction, m)
    torch.cuda.synchronize()
    eng.check()
    return out.float().cpu()


def _assert_parity(got, ref, what=""):
    err = (got - ref).abs()
    b1, b2 = cp1_bound(ref), tolerance_bound(ref)
    v1, v2 = int((err > b1).sum()), int((err > b2).sum())
    rel = (err / ref.abs().clamp_min(1e-3)).max().item()
    assert not torch.isnan(got).any(), f"{what}: NaN in output"
    assert v1 == 0 and v2 == 0, (f"{what}: {v1} elements beyond the cp=1 bound, {v2} beyond the distributed bound; "
                                 f"max|err|={err.max().item():.5f} max rel={rel:.4f} max|ref|={ref.abs().max().item():.4f}")


# ------------------------------------------------------------------------------------------------
# golden vectors of the reference's own trimul_ref
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(CASES))
def test_forward_matches_reference_golden(name, golden):
    kw = dict(CASES[name])
    direction = kw.pop("direction")
    case = bf16_round_case(make_case(**kw))
    got = _run(case, direction)
    _assert_parity(got, torch.from_numpy(golden[name]), name)


# ------------------------------------------------------------------------------------------------
# oracle on seeded inputs: directions x bias x mask x shapes (edge shapes included)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
@pytest.mark.parametrize("B,N,D,bias,mask", [
    (1, 8, 128, "none", "none"),        # smallest legal token extent
    (1, 72, 128, "all", "random"),      # not a multiple of any tile
    (2, 136, 128, "out", "pad"),        # batch > 1, ragged tiles, padding mask
    (1, 200, 256, "all", "ones"),       # D=256, ragged
    (2, 64, 256, "none", "random"),
    (1, 256, 128, "all", "random"),     # the reference's own parity shape (N=256, D=128)
    (1, 136, 384, "all", "random"),     # wide rows: six gated chunks, three output-gate chunks, ragged tiles
    (2, 72, 512, "out", "pad"),         # D=512: one staging buffer, single accumulator in the output projection
    (1, 264, 512, "all", "ones"),       # D=512, more than two tiles per line
])
def test_forward_matches_oracle(direction, B, N, D, bias, mask):
    case = bf16_round_case(make_case(B, N, D, seed=1000 + N + D, bias=bias, mask=mask))
    ref = trimul_oracle(case["x"], direction, case["mask"], eps=1e-5, **weights_of(case))
    _assert_parity(_run(case, direction), ref, f"{direction} B{B} N{N} D{D} {bias} {mask}")


def test_reference_cpu_config_shape():
    """configs[0] of the benchmark definition: (1,256,256,128), gamma=1, beta=0, biases 0, mask ones."""
    case = bf16_round_case(make_case(1, 256, 128, seed=0, ln_affine=False, bias="none", mask="ones"))
    ref = trimul_oracle(case["x"], "outgoing", case["mask"], **weights_of(case))
    _assert_parity(_run(case, "outgoing"), ref, "config0")


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_single_gpu_config_shape_against_gpu_evaluated_oracle(direction):
    """configs[1]: (1,1024,1024,128) with LayerNorm affine and biases on all six projections.  The
    fp32 oracle at this size is evaluated by the same oracle code on CUDA fp32 tensors (TF32 off)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    case = bf16_round_case(make_case(1, 1024, 128, seed=1, bias="all", mask="ones"))
    cg = {k: (None if v is None else v.to(DEV)) for k, v in case.items()}
    ref = trimul_oracle(cg["x"], direction, cg["mask"], **{k: cg[k] for k in weights_of(case)}).cpu()
    del cg
    torch.cuda.empty_cache()
    _assert_parity(_run(case, direction), ref, f"config1 {direction}")


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_larger_shape_against_the_streamed_tiled_oracle(direction):
    """N=768, D=256: the fp32 oracle is never materialised -- the tiled oracle (the reference's
    ``trimul_ref_chunked`` form) runs on the GPU in fp32 (TF32 off) and every block is compared as it is made."""
    from oracle.trimul_oracle import trimul_oracle_tiled

    torch.backends.cuda.matmul.allow_tf32 = False
    case = bf16_round_case(make_case(1, 768, 256, seed=41, bias="all", mask="pad"))
    got = _run(case, direction).to(DEV)
    cg = {k: (None if v is None else v.to(DEV)) for k, v in case.items()}
    count = {"beyond": 0, "far_beyond": 0, "beyond_cp1": 0, "max": 0.0}

    def on_tile(i0, i1, j0, j1, ref):
        err = (got[:, i0:i1, j0:j1] - ref).abs()
        bound = 2e-2 + 6e-2 * ref.abs()
        count["beyond"] += int((err > bound).sum())
        count["far_beyond"] += int((err > 1.5 * bound).sum())
        count["beyond_cp1"] += int((err > 0.01 * ref.abs().max() + 0.01 * ref.abs()).sum())
        count["max"] = max(count["max"], err.max().item())

    trimul_oracle_tiled(cg["x"], direction, cg["mask"], row_tile=256, on_tile=on_tile, **{k: cg[k] for k in weights_of(case)})
    # 1.5e8 output elements, each carrying four bf16 roundings along the chain: the tail of that rounding error
    # crosses a fixed absolute bound written for tests of <= 1e6 elements about once per 1e8 elements (|err| =
    # 0.024 against 0.02 + 0.06 |ref| at an element with |ref| < 0.07 was seen).  Allowed: two such elements per
    # 1e8, none beyond 1.5 x the bound, none beyond the cp=1 bound (which scales with the block's max |ref|).
    allowed = -(-got.numel() * 2 // 10 ** 8)
    assert count["beyond"] <= allowed and count["far_beyond"] == 0 and count["beyond_cp1"] == 0, count


def test_off_centre_rows():
    """Rows whose mean is far from zero (|mean| >> std) must not lose the LayerNorm signal
    (the reference pins this for its own chains: tests/workflows/test_trimul_autotune.py:611-633)."""
    case = make_case(1, 64, 128, seed=9, bias="all", mask="none")
    case["x"] = case["x"] + 40.0 * torch.randn(1, 64, 64, 1, generator=torch.Generator().manual_seed(4))
    case = bf16_round_case(case)
    ref = trimul_oracle(case["x"], "outgoing", None, **weights_of(case))
    _assert_parity(_run(case, "outgoing"), ref, "off-centre")


# ------------------------------------------------------------------------------------------------
# size-independent properties (also used at full benchmark sizes by bench.py --verify)
# ------------------------------------------------------------------------------------------------
def test_deterministic_and_mask_of_ones_is_identity():
    case = bf16_round_case(make_case(1, 128, 128, seed=5, bias="all", mask="ones"))
    a = _run(case, "outgoing")
    b = _run(case, "outgoing")
    assert torch.equal(a, b)
    nomask = dict(case, mask=None)
    assert torch.equal(a, _run(nomask, "outgoing"))
    for dt in (torch.bfloat16, torch.bool, torch.uint8):
        assert torch.equal(a, _run(case, "outgoing", mask_dtype=dt))


def test_batch_planes_are_independent():
    case = bf16_round_case(make_case(2, 96, 128, seed=6, bias="all", mask="random"))
    both = _run(case, "incoming")
    for b in range(2):
        one = dict(case, x=case["x"][b:b + 1].contiguous(), mask=case["mask"][b:b + 1].contiguous())
        assert torch.equal(both[b:b + 1], _run(one, "incoming"))


def test_zero_mask_kills_the_contraction_only():
    """mask = 0 zeroes a|b, hence tri; the output is then gate * (beta_out . W^T + b), with the gate
    untouched by the mask."""
    case = bf16_round_case(make_case(1, 64, 128, seed=7, bias="all", mask="ones"))
    case["mask"] = torch.zeros_like(case["mask"])
    ref = trimul_oracle(case["x"], "outgoing", case["mask"], **weights_of(case))
    assert ref.abs().max() > 1e-3
    _assert_parity(_run(case, "outgoing"), ref, "zero mask")


def test_incoming_is_outgoing_of_the_transposed_pair_tensor():
    """tri_in(x) == tri_out(x^T): checked on the contraction kernel's operand planes and output."""
    from fold_cp_ops_b200 import kernels as K

    B, N, D = 1, 96, 128
    case = bf16_round_case(make_case(B, N, D, seed=8, bias="all", mask="random"))
    eng = _engine(case)
    W = eng.weights

    def planes(x, m, direction):
        ab = torch.empty((2, D, B, N, N), dtype=torch.bfloat16, device=DEV)
        gate = torch.empty((B, N, N, D), dtype=torch.bfloat16, device=DEV)
        tri = torch.empty((D, B, N, N), dtype=torch.bfloat16, device=DEV)
        g = K.make_geom(B, N, D, direction, 1e-5)
        K.ln_gated_proj(g, x, m, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, [ab.data_ptr()], gate, eng.status)
        K.tri_contract(g, ab, [tri.data_ptr()], eng.status)
        torch.cuda.synchronize()
        return ab.cpu(), tri.cpu()

    x = case["x"].to(DEV).bfloat16()
    m = case["mask"].to(DEV)
    ab_in, tri_in = planes(x, m, "incoming")
    ab_out, tri_out = planes(x.transpose(1, 2).contiguous(), m.transpose(1, 2).contiguous(), "outgoing")
    assert torch.equal(ab_in, ab_out)
    assert torch.equal(tri_in, tri_out)
    eng.check()


# ------------------------------------------------------------------------------------------------
# single kernels against the oracle with bf16 rounding at the same points
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
@pytest.mark.parametrize("D,N,B", [(128, 72, 1), (256, 40, 2), (384, 40, 1), (512, 24, 2)])
def test_kernel_ln_gated_proj(direction, D, N, B):
    from fold_cp_ops_b200 import kernels as K

    case = bf16_round_case(make_case(B, N, D, seed=11, bias="all", mask="random"))
    eng = _engine(case)
    W = eng.weights
    ab = torch.full((2, D, B, N, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    gate = torch.full((B, N, N, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    g = K.make_geom(B, N, D, direction, 1e-5)
    K.ln_gated_proj(g, case["x"].to(DEV).bfloat16(), case["mask"].to(DEV), W.norm_in_w, W.norm_in_b, W.w_packed,
                    W.bias_packed, [ab.data_ptr()], gate, eng.status)
    torch.cuda.synchronize()
    eng.check()
    s = trimul_stages(case["x"], direction, case["mask"], **weights_of(case), round_bf16=True)
    for h, key in ((0, "a"), (1, "b")):
        want = s[key].permute(3, 0, 1, 2)
        if direction == "incoming":
            want = want.transpose(2, 3)
        err = (ab[h].float().cpu() - want).abs()
        assert (err <= 0.02 + 0.02 * want.abs()).all(), (key, err.max().item())
    err = (gate.float().cpu() - s["gate"]).abs()
    assert (err <= 0.01).all(), err.max().item()


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
@pytest.mark.parametrize("D,cp0,cp1,N,B", [
    (128, 8, 1, 64, 1),    # 16 channels per rank: the smallest store box
    (256, 8, 1, 64, 2),    # the eight-rank split of the headline width: 32 channels per rank
    (384, 8, 1, 64, 1),    # 48 channels per rank: owner boundaries fall inside a 64-channel group
    (512, 8, 1, 128, 1),   # 64 channels per rank, wide-row kernels
    (256, 2, 4, 64, 1),    # 2-D grid, rows x columns
    (128, 4, 2, 64, 2),
    (384, 2, 2, 48, 1),
    (256, 4, 1, 96, 1),
    (256, 2, 1, 48, 2),
    (128, 2, 1, 768, 1),   # several contraction tiles per plane: each rank's tile walk starts at its own block
    (128, 2, 2, 768, 1),
])
def test_every_rank_of_a_cp_grid_run_in_turn_on_one_gpu(direction, D, cp0, cp1, N, B):
    """The cp > 1 data path without a second GPU: every rank's kernels are launched one after the other
    on this GPU through the stateless entry points, with the peers' receive buffers being plain local
    allocations.  No kernel waits on another (all projections finish before the first contraction
    starts, all contractions before the first output kernel), so this covers the owner arithmetic and
    the store boxes of both fused reshards for every rank of the grid -- eight ranks included -- and
    is compared with the fp32 oracle on the global tensor."""
    from fold_cp_ops_b200 import kernels as K

    cp = cp0 * cp1
    case = bf16_round_case(make_case(B, N, D, seed=D + 10 * cp0 + cp1, bias="all", mask="random"))
    eng = _engine(case)
    W = eng.weights
    x = case["x"].to(DEV).bfloat16()
    mask = case["mask"].to(DEV)
    ni, nj = N // cp0, N // cp1
    geoms = [K.make_geom(B, N, D, direction, 1e-5, cp0, cp1, r) for r in range(cp)]
    ws = K.workspace_bytes(geoms[0])
    nan16 = lambda nbytes: torch.full((nbytes // 2,), float("nan"), dtype=torch.bfloat16, device=DEV)
    ab = [nan16(ws.ab_bytes) for _ in range(cp)]
    tri = [nan16(ws.tri_bytes) for _ in range(cp)]
    gate = [nan16(ws.gate_bytes) for _ in range(cp)]
    block = lambda t, r: t[:, (r // cp1) * ni:(r // cp1 + 1) * ni, (r % cp1) * nj:(r % cp1 + 1) * nj].contiguous()
    for r, g in enumerate(geoms):
        K.ln_gated_proj(g, block(x, r), block(mask, r), W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed,
                        [t.data_ptr() for t in ab], gate[r], eng.status)
    torch.cuda.synchronize()
    eng.check()
    for r, g in enumerate(geoms):
        assert not torch.isnan(ab[r]).any(), f"rank {r}: part of its a|b planes was never written"
        K.tri_contract(g, ab[r], [t.data_ptr() for t in tri], eng.status)
    torch.cuda.synchronize()
    eng.check()
    out = torch.full_like(x, float("nan"))
    for r, g in enumerate(geoms):
        assert not torch.isnan(tri[r]).any(), f"rank {r}: part of its contraction input was never written"
        out_r = torch.full((B, ni, nj, D), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.ln_out_proj(g, tri[r], gate[r], W.w_fold, W.cd, out_r, eng.status)
        out[:, (r // cp1) * ni:(r // cp1 + 1) * ni, (r % cp1) * nj:(r % cp1 + 1) * nj] = out_r
    torch.cuda.synchronize()
    eng.check()
    ref = trimul_oracle(case["x"], direction, case["mask"], eps=1e-5, **weights_of(case))
    _assert_parity(out.float().cpu(), ref, f"cp{cp0}x{cp1} D={D} {direction}")
    one = eng.forward(x, direction, mask)
    torch.cuda.synchronize()
    # the same arithmetic per element as the one-rank forward (only the partition differs)
    assert (out.float() - one.float()).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("N,planes_d", [(8, 128), (64, 128), (200, 128), (1024, 128)])
def test_kernel_tri_contract(N, planes_d):
    from fold_cp_ops_b200 import kernels as K

    torch.manual_seed(N)
    D, B = planes_d, 1
    ab = (0.5 * torch.randn(2, D, B, N, N, device=DEV)).to(torch.bfloat16)
    tri = torch.full((D, B, N, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    st = K.new_status(DEV)
    K.tri_contract(K.make_geom(B, N, D, "outgoing", 1e-5), ab, [tri.data_ptr()], st)
    torch.cuda.synchronize()
    K.check_status(st)
    torch.backends.cuda.matmul.allow_tf32 = False
    want = torch.bmm(ab[0, :, 0].float(), ab[1, :, 0].float().transpose(1, 2))
    err = (tri[:, 0].float() - want).abs()
    # fp32 accumulation of exact bf16 products, one bf16 rounding of the result
    assert (err <= 2.0 ** -8 * want.abs() + 1e-3 * want.abs().max()).all(), err.max().item()


@pytest.mark.parametrize("N", [8, 200, 512])
def test_kernel_tri_contract_pair_form_equals_single_cta_form(N):
    """The default contraction kernel works on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles); the
    single-CTA 128 x 256 kernel is a tuning choice.  Same K order, same fp32 accumulation: bitwise equal."""
    from fold_cp_ops_b200 import kernels as K

    torch.manual_seed(7 + N)
    D = 128
    ab = (0.5 * torch.randn(2, D, 1, N, N, device=DEV)).to(torch.bfloat16)
    outs = []
    for form in ("pair", "single", "auto"):
        tri = torch.full((D, 1, N, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        st = K.new_status(DEV)
        K.tri_contract(K.make_geom(1, N, D, "outgoing", 1e-5), ab, [tri.data_ptr()], st, tuning=K.make_tuning(form))
        torch.cuda.synchronize()
        K.check_status(st)
        outs.append(tri)
    assert not torch.isnan(outs[0].float()).any()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    with pytest.raises(ValueError, match="contract_form"):
        K.make_tuning("triple")


@pytest.mark.parametrize("form", ["pair", "single"])
@pytest.mark.parametrize("N,band", [(200, 2), (600, 2), (1024, 3), (1024, 8), (1280, 4)])
def test_kernel_tri_contract_banded_tile_walk_equals_row_major(N, band, form):
    """The order in which the tiles of a plane are walked (bands of `band` tile rows, column by column
    inside a band; bands that do not divide the tile grid included) changes which CTA computes which tile
    and nothing else; the pacing of the CTA pairs (off, the library's 20 us, 50 us) changes only WHEN a pair
    starts a tile.  Every combination is bitwise equal to the unpaced row-major walk."""
    from fold_cp_ops_b200 import kernels as K

    torch.manual_seed(N + band)
    D = 128
    ab = (0.5 * torch.randn(2, D, 1, N, N, device=DEV)).to(torch.bfloat16)
    outs = []
    for rows, pace in ((1, -1), (band, 0), (band, 50000)):
        tri = torch.full((D, 1, N, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        st = K.new_status(DEV)
        g = K.make_geom(1, N, D, "outgoing", 1e-5)
        K.tri_contract(g, ab, [tri.data_ptr()], st,
                       tuning=K.make_tuning(form, contract_band_rows=rows, contract_pace_ns=pace))
        torch.cuda.synchronize()
        K.check_status(st)
        outs.append(tri)
    assert not torch.isnan(outs[0].float()).any()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("D,B,n,offset", [(128, 1, 8, 0.5), (128, 1, 72, 0.5), (256, 2, 40, 0.5), (256, 1, 64, 30.0),
                                          (384, 1, 40, 0.5), (512, 2, 24, 0.5), (512, 1, 72, 0.5)])
def test_kernel_ln_out_proj(D, B, n, offset):
    """The folded LayerNorm (rstd * (x W'^T - mean c) + d) against an explicit fp32 LayerNorm; the last
    case shifts every token's channels far off zero (|mean| = 10 sigma), where the fold subtracts two
    large numbers."""
    from fold_cp_ops_b200 import kernels as K

    rows = B * n * n
    torch.manual_seed(rows)
    tri = (3.0 * torch.randn(D, rows, device=DEV) + offset).to(torch.bfloat16)
    gate = torch.rand(rows, D, device=DEV).to(torch.bfloat16)
    lw = (1 + 0.1 * torch.randn(D, device=DEV)).float()
    lb = (0.1 * torch.randn(D, device=DEV)).float()
    w = (torch.randn(D, D, device=DEV) / D ** 0.5).to(torch.bfloat16)
    bo = (0.02 * torch.randn(D, device=DEV)).float()
    out = torch.full((rows, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    st = K.new_status(DEV)
    w_fold, cd = K.pack_out_weights(D, w, lw, lb, bo)
    K.ln_out_proj(K.make_geom(B, n, D, "outgoing", 1e-5), tri, gate, w_fold, cd, out, st)
    torch.cuda.synchronize()
    K.check_status(st)
    torch.backends.cuda.matmul.allow_tf32 = False
    trin = layer_norm(tri.float().t(), lw, lb, 1e-5)
    want = (trin @ w.float().t() + bo) * gate.float()
    err = (out.float() - want).abs()
    tol = 0.03 + 0.02 * want.abs() if offset < 1 else 0.08 + 0.03 * want.abs()
    assert (err <= tol).all(), err.max().item()


# ------------------------------------------------------------------------------------------------
# the single-GPU front doors and their refusals
# ------------------------------------------------------------------------------------------------
def test_trimul_autotuned_front_door_and_dtype_roundtrip():
    from fold_cp_ops_b200.workflows.trimul_autotune import trimul_autotuned

    case = bf16_round_case(make_case(1, 64, 128, seed=12, bias="all", mask="random"))
    w = {k: (None if v is None else v.to(DEV)) for k, v in weights_of(case).items()}
    ref = trimul_oracle(case["x"], "incoming", case["mask"], **weights_of(case))
    for dt in (torch.bfloat16, torch.float32):
        x = case["x"].to(DEV).to(dt)
        got = trimul_autotuned(x, **w, mask=case["mask"].to(DEV), direction="incoming")
        assert got.dtype is dt and got.shape == x.shape
        _assert_parity(got.float().cpu(), ref, f"front door {dt}")
    buf = torch.empty_like(x)
    assert trimul_autotuned(x, **w, direction="incoming", out=buf) is buf


def test_refusals():
    from fold_cp_ops_b200.workflows.trimul_autotune import trimul_autotuned

    case = make_case(1, 16, 128, seed=13)
    w = {k: (None if v is None else v.to(DEV)) for k, v in weights_of(case).items()}
    x = case["x"].to(DEV).bfloat16()
    with pytest.raises(ValueError, match="direction"):
        trimul_autotuned(x, **w, direction="sideways")
    with pytest.raises(ValueError, match="select"):
        trimul_autotuned(x, **w, select="fastest")
    with pytest.raises(ValueError, match="16-byte aligned"):
        trimul_autotuned(x[:, :12, :12].contiguous(), **w)
    with pytest.raises(ValueError, match="square"):
        trimul_autotuned(x[:, :8].contiguous(), **w)
    with pytest.raises(ValueError, match="float32"):
        trimul_autotuned(x, **dict(w, norm_in_w=w["norm_in_w"].bfloat16()))
    with pytest.raises(ValueError, match=r"\(2D, D\)"):
        trimul_autotuned(x, **dict(w, p_in_w=w["p_in_w"][:128]))
    with pytest.raises(ValueError, match="mask"):
        trimul_autotuned(x, **w, mask=torch.ones(1, 8, 8, device=DEV))
    case64 = make_case(1, 16, 64, seed=14)
    w64 = {k: (None if v is None else v.to(DEV)) for k, v in weights_of(case64).items()}
    with pytest.raises(ValueError, match="not supported"):
        trimul_autotuned(case64["x"].to(DEV).bfloat16(), **w64)


def test_module_front_door_cp1_plain_tensor_and_one_device_mesh():
    import torch.nn as nn

    from fold_cp_ops_b200.distributed.trimul_weights import trimul_module_from_weights
    from fold_cp_ops_b200.distributed.workflows.trimul_autotuned import TriangularMultiplication

    case = bf16_round_case(make_case(1, 64, 128, seed=15, bias="out", mask="random"))
    layer = trimul_module_from_weights({k: (None if v is None else v.to(DEV)) for k, v in weights_of(case).items()})
    mod = TriangularMultiplication(layer, "outgoing", None, None)
    assert mod.incoming_variant == "cp1_fallback" and mod.prepare(n_token=64) is None
    x = case["x"].to(DEV).bfloat16()
    got = mod(x, case["mask"].to(DEV))
    assert isinstance(got, torch.Tensor) and got.dtype is torch.bfloat16
    ref = trimul_oracle(case["x"], "outgoing", case["mask"], **weights_of(case))
    _assert_parity(got.float().cpu(), ref, "module cp1")
    mod.free()


# ------------------------------------------------------------------------------------------------
# bounded waits: a wait that nothing satisfies ends with a status, not a hang
# ------------------------------------------------------------------------------------------------
def test_expired_wait_reports_status_and_context_survives():
    from fold_cp_ops_b200 import kernels as K

    flags = torch.zeros(16, dtype=torch.int64, device=DEV)
    st = K.new_status(DEV)
    K.peer_wait(flags, 3, 1, st, timeout_ns=20_000_000)  # 20 ms; nobody signals slot 3
    torch.cuda.synchronize()
    from fold_cp_ops_b200.distributed import CollectiveError

    with pytest.raises(K.DeviceWaitTimeout, match="cross-rank flag wait expired") as info:
        K.check_status(st)
    assert isinstance(info.value, CollectiveError)
    # the status was cleared and the context still works: a satisfied wait passes
    K.peer_signal([flags.data_ptr()], 3)
    K.peer_wait(flags, 3, 1, st, timeout_ns=20_000_000)
    torch.cuda.synchronize()
    K.check_status(st)
    assert int(flags[3].item()) == 1


def test_engine_raises_on_the_next_forward_after_a_wait_gave_up():
    """A forward whose status record shows an expired wait must not go unnoticed by a caller of the
    public API: the next forward (and ``check``) raise ``DeviceWaitTimeout``."""
    from fold_cp_ops_b200 import kernels as K

    case = bf16_round_case(make_case(1, 32, 128, seed=21, bias="none", mask="none"))
    eng = _engine(case)
    x = case["x"].to(DEV).bfloat16()
    eng.forward(x, "outgoing")
    flags = torch.zeros(16, dtype=torch.int64, device=DEV)
    K.peer_wait(flags, 1, 1, eng.status, timeout_ns=10_000_000)   # a wait nothing satisfies, on the engine's record
    eng.forward(x, "outgoing")                                     # mirrors the record to the host
    torch.cuda.synchronize()
    with pytest.raises(K.DeviceWaitTimeout, match="BACK"):
        eng.forward(x, "outgoing")
    eng.forward(x, "outgoing")   # the record was cleared: the engine works again
    torch.cuda.synchronize()
    eng.check()


# ------------------------------------------------------------------------------------------------
# plans, tuning, statistics, the one-batch-plane path, the functional front door
# ------------------------------------------------------------------------------------------------
def test_plan_path_equals_stateless_entry_points():
    """The engine launches through a plan (descriptors encoded once); the stateless per-kernel entry
    points encode them per call.  Same kernels, same arguments: bitwise equal, also on the second use
    of the plan with another output buffer."""
    from fold_cp_ops_b200 import kernels as K

    B, N, D = 2, 72, 128
    case = bf16_round_case(make_case(B, N, D, seed=22, bias="all", mask="random"))
    eng = _engine(case)
    W = eng.weights
    x = case["x"].to(DEV).bfloat16()
    m = case["mask"].to(DEV)
    for direction in ("outgoing", "incoming"):
        ab = torch.empty((2, D, B, N, N), dtype=torch.bfloat16, device=DEV)
        tri = torch.empty((D, B, N, N), dtype=torch.bfloat16, device=DEV)
        gate = torch.empty((B, N, N, D), dtype=torch.bfloat16, device=DEV)
        want = torch.empty_like(x)
        K.forward_single(K.make_geom(B, N, D, direction, 1e-5), x, m, W.norm_in_w, W.norm_in_b, W.w_packed,
                         W.bias_packed, W.w_fold, W.cd, ab, tri, gate, want, eng.status)
        got1 = eng.forward(x, direction, m)
        got2 = eng.forward(x, direction, m)
        torch.cuda.synchronize()
        eng.check()
        assert torch.equal(got1, want) and torch.equal(got2, want)


def test_one_batch_plane_at_a_time_equals_full_batch(monkeypatch):
    """``CPO_TRIMUL_WORKSPACE_BYTES`` smaller than the full-batch workspace makes the cp=1 engine run one
    batch plane per launch (what B=2, N=8192, D=128 needs on one GPU); batch planes are independent, so
    the result is the same as the full-batch run and inside the oracle bound."""
    case = bf16_round_case(make_case(2, 80, 128, seed=23, bias="all", mask="pad"))
    ref = trimul_oracle(case["x"], "incoming", case["mask"], **weights_of(case))
    full = _run(case, "incoming")
    monkeypatch.setenv("CPO_TRIMUL_WORKSPACE_BYTES", "1")
    eng = _engine(case)
    out = eng.forward(case["x"].to(DEV).bfloat16(), "incoming", case["mask"].to(DEV))
    torch.cuda.synchronize()
    eng.check()
    assert next(iter(eng._ws.values())).planes_b == 1
    assert torch.equal(out.float().cpu(), full)
    _assert_parity(out.float().cpu(), ref, "one batch plane per launch")


def test_workspace_cache_is_fifo_and_results_survive_eviction(monkeypatch):
    monkeypatch.setenv("CPO_TRIMUL_RECV_CACHE", "1")
    case_a = bf16_round_case(make_case(1, 32, 128, seed=24, bias="none", mask="none"))
    eng = _engine(case_a)
    xa = case_a["x"].to(DEV).bfloat16()
    xb = xa[:, :24, :24].contiguous()
    a1 = eng.forward(xa, "outgoing")
    assert list(eng._ws) == [(1, 32)]
    eng.forward(xb, "outgoing")
    assert list(eng._ws) == [(1, 24)]          # the older workspace was evicted
    a2 = eng.forward(xa, "outgoing")
    torch.cuda.synchronize()
    eng.check()
    assert list(eng._ws) == [(1, 32)] and torch.equal(a1, a2)


def test_last_forward_stats_reports_kernel_times_and_spans():
    case = bf16_round_case(make_case(1, 256, 128, seed=25, bias="none", mask="ones"))
    eng = _engine(case)
    x = case["x"].to(DEV).bfloat16()
    eng.forward(x, "outgoing")
    eng.collect_stats = True
    eng.forward(x, "outgoing")
    st = eng.last_forward_stats()
    assert set(st["stage_ms"]) == {"ln_gated_proj", "tri_contract", "ln_out_proj"}
    assert all(v > 0 for v in st["stage_ms"].values())
    assert st["wait_ms"] == {}                          # cp = 1: no cross-rank waits
    sp = st["span_ms"]
    assert 0 < sp["ln_gated_proj"] <= sp["forward"] and 0 < sp["tri_contract"] and 0 < sp["ln_out_proj"]
    assert 0 <= sp["first_store_after_start"] <= sp["ln_gated_proj"]
    assert st["bytes_to_peers"] == {"front": 0, "back": 0}


def test_trimul_a2a_functional_front_door_on_one_gpu():
    """``trimul_a2a`` with a plain tensor (or a one-device mesh) routes to the single-GPU chain."""
    from fold_cp_ops_b200.distributed.workflows.trimul_autotuned import trimul_a2a

    case = bf16_round_case(make_case(1, 64, 128, seed=26, bias="all", mask="random"))
    w = {k: (None if v is None else v.to(DEV)) for k, v in weights_of(case).items()}
    for direction in ("outgoing", "incoming"):
        ref = trimul_oracle(case["x"], direction, case["mask"], **weights_of(case))
        got = trimul_a2a(case["x"].to(DEV).bfloat16(), w, torch.bfloat16, direction=direction, mask=case["mask"].to(DEV))
        _assert_parity(got.float().cpu(), ref, f"trimul_a2a {direction}")
    with pytest.raises(TypeError, match="unknown fused_kwargs"):
        trimul_a2a(case["x"].to(DEV).bfloat16(), w, torch.bfloat16, back_cluster=2)
