"""The allocation-free forward (``trimul_sm100_forward_static``) against the regular entry point.

Some hosts of the library cannot give it freshly allocated device memory -- a server whose pool
already owns the GPU, a sandboxed plugin, a loop that cannot afford cudaMalloc's synchronisation --
so this entry point keeps its scratch in a 32 MiB array inside the library.  The test drives it
through the C ABI twice in a row (the second call finds the first call's leftovers in the shared
array) and expects exactly the output of ``trimul_sm100_forward`` with caller-provided buffers; it
also checks that a shape beyond the built-in capacity is refused with a clear message.  The file
name sorts last so that a stop-at-first-failure run has already executed every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(B, N, D, seed):
    from fold_cp_ops_b200 import kernels as K
    from fold_cp_ops_b200.engine import PackedWeights
    from oracle.trimul_oracle import bf16_round_case, make_case, weights_of

    dev = torch.device("cuda:0")
    case = bf16_round_case(make_case(B, N, D, seed=seed, bias="all", mask="random"))
    W = PackedWeights({k: (None if v is None else v.to(dev)) for k, v in weights_of(case).items()}, dev)
    x = case["x"].to(dev).bfloat16().contiguous()
    m = case["mask"].to(dev).contiguous()
    return K, dev, case, W, x, m


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_static_scratch_forward_matches_regular_forward_twice(direction):
    B, N, D = 1, 96, 128
    K, dev, case, W, x, m = _setup(B, N, D, seed=77)
    geom = K.make_geom(B, N, D, direction, 1e-5)
    st = K.new_status(dev)
    # regular entry point with caller-provided scratch
    ab = torch.empty((2, D, B, N, N), dtype=torch.bfloat16, device=dev)
    tri = torch.empty((D, B, N, N), dtype=torch.bfloat16, device=dev)
    gate = torch.empty((B, N, N, D), dtype=torch.bfloat16, device=dev)
    want = torch.empty_like(x)
    K.forward_single(geom, x, m, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, W.w_fold, W.cd, ab, tri, gate,
                     want, st)
    torch.cuda.synchronize()
    K.check_status(st)
    # the allocation-free entry point, two calls in a row on different inputs then the same input
    other = torch.flip(x, dims=(1,)).contiguous()
    scratch_out = torch.empty_like(x)
    K.forward_static(geom, other, m, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, W.w_fold, W.cd, scratch_out, st)
    got = []
    for _ in range(2):
        out = torch.full_like(x, float("nan"))
        K.forward_static(geom, x, m, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, W.w_fold, W.cd, out, st)
        got.append(out)
    torch.cuda.synchronize()
    K.check_status(st)
    for out in got:
        assert not torch.isnan(out).any()
        # same kernels, same inputs, only the scratch location differs: the tolerance is exact equality
        assert torch.equal(out, want), (out.float() - want.float()).abs().max().item()


def test_static_scratch_accepts_the_exact_capacity_shape():
    """B=1, N=128, D=256 needs 8 * 128 * 128 * 256 bytes = exactly the 32 MiB the array holds."""
    from fold_cp_ops_b200 import _lib

    B, N, D = 1, 128, 256
    assert 8 * B * N * N * D == _lib.STATIC_SCRATCH_BYTES
    K, dev, case, W, x, m = _setup(B, N, D, seed=79)
    geom = K.make_geom(B, N, D, "outgoing", 1e-5)
    st = K.new_status(dev)
    ab = torch.empty((2, D, B, N, N), dtype=torch.bfloat16, device=dev)
    tri = torch.empty((D, B, N, N), dtype=torch.bfloat16, device=dev)
    gate = torch.empty((B, N, N, D), dtype=torch.bfloat16, device=dev)
    want = torch.empty_like(x)
    K.forward_single(geom, x, m, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, W.w_fold, W.cd, ab, tri, gate,
                     want, st)
    got = torch.full_like(x, float("nan"))
    K.forward_static(geom, x, m, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, W.w_fold, W.cd, got, st)
    torch.cuda.synchronize()
    K.check_status(st)
    assert torch.equal(got, want)


def test_static_scratch_refuses_shapes_beyond_its_capacity():
    from fold_cp_ops_b200 import _lib

    B, N, D = 1, 136, 256   # 8 * 136 * 136 * 256 bytes = 36.1 MiB > 32 MiB
    K, dev, case, W, x, m = _setup(B, 8, D, seed=78)
    geom = K.make_geom(B, N, D, "outgoing", 1e-5)
    assert 8 * B * N * N * D > _lib.STATIC_SCRATCH_BYTES
    xb = torch.zeros((B, N, N, D), dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError, match="needs .* bytes of scratch but the built-in array holds"):
        K.forward_static(geom, xb, None, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, W.w_fold, W.cd,
                         torch.empty_like(xb), K.new_status(dev))
    geom2 = K.make_geom(B, 64, D, "outgoing", 1e-5, cp0=2, cp1=1, rank=0)
    with pytest.raises(ValueError, match="single-GPU only"):
        K.forward_static(geom2, xb, None, W.norm_in_w, W.norm_in_b, W.w_packed, W.bias_packed, W.w_fold, W.cd,
                         torch.empty_like(xb), K.new_status(dev))
