"""Host-side logic that needs no GPU: layouts, peer map, sharding validation, weight adapters,
tuning surface, the public front door's construction-time behaviour, the C ABI's symbols and the
index arithmetic of the two fused reshards (all ranks simulated in one process)."""
import ctypes
import inspect
from types import SimpleNamespace

import numpy as np
import pytest
import torch
import torch.nn as nn

from fold_cp_ops_b200 import _lib
from fold_cp_ops_b200 import kernels as K
from fold_cp_ops_b200.distributed import (LayoutLeftMap, LayoutMap, LayoutRightMap, PeMap, W_KEYS, W_PROJ_BIAS_KEYS,
                                          weights_from_trimul_module)
from fold_cp_ops_b200.distributed.dtensor_adapter import (_effective_placements, _is_dtensor, _rowmaj_stride,
                                                          _token_split_factor, validate_trimul_sharding)
from fold_cp_ops_b200.distributed.trimul_weights import trimul_module_from_weights
from fold_cp_ops_b200.distributed.workflows import trimul_autotuned as front
from fold_cp_ops_b200.distributed.workflows.trimul_tuning import (BackTuning, FrontTuning, NOT_EXPOSED, TriMulTuning)


class Shard:
    def __init__(self, dim):
        self.dim = dim

    def is_shard(self):
        return True

    def __eq__(self, o):
        return isinstance(o, Shard) and o.dim == self.dim

    def __repr__(self):
        return f"Shard({self.dim})"


class Replicate:
    def is_shard(self):
        return False

    def __repr__(self):
        return "Replicate()"


def fake_mesh(shape):
    n = int(np.prod(shape))
    return SimpleNamespace(mesh=torch.arange(n).reshape(shape), ndim=len(shape))


# ------------------------------------------------------------------------------------------------
# layout maps
# ------------------------------------------------------------------------------------------------
def test_layout_right_left_roundtrip():
    r = LayoutRightMap((2, 3, 4))
    l = LayoutLeftMap((2, 3, 4))
    assert r.strides == (12, 4, 1) and l.strides == (1, 2, 6)
    for lay in (r, l):
        assert lay.is_unique and lay.is_exhaustive and lay.numel == 24 and lay.required_span_size == 24
        for f in range(24):
            assert lay(lay.unravel(f)) == f
    assert r.ravel((1, 2, 3)) == 23


def test_layout_slicing_and_errors():
    lay = LayoutMap((12, 4, 1), (2, 3, 4))
    sub = lay[1:, :, 2]
    assert sub.shape == (1, 3) and sub.offset == 14 and sub.strides == (12, 4)
    assert lay[:, 1].shape == (2, 4)
    assert not LayoutMap((24, 4, 1), (2, 3, 4)).is_exhaustive
    with pytest.raises(ValueError, match="unique"):
        LayoutMap((1, 1), (2, 2))
    with pytest.raises(ValueError, match="zero values"):
        LayoutMap((3, 1), (0, 3))
    with pytest.raises(ValueError, match="same length"):
        LayoutMap((1,), (2, 2))
    with pytest.raises(ValueError):
        lay((2, 0, 0))
    with pytest.raises(TypeError):
        lay.unravel(1.5)
    with pytest.raises(ValueError, match="Negative or zero steps"):
        lay[::-1]
    with pytest.raises(ValueError, match="unmapped|out of the valid range"):
        LayoutMap((24, 4, 1), (2, 3, 4)).unravel(13)


# ------------------------------------------------------------------------------------------------
# peer map
# ------------------------------------------------------------------------------------------------
def test_pe_map_1d_and_2d_and_dp():
    pm = PeMap.from_mesh_placements(fake_mesh((4,)), [Shard(1)], my_rank=2, device=torch.device("cpu"))
    assert (pm.cp, pm.my_cp_rank, pm.cp_pe_table.tolist()) == (4, 2, [0, 1, 2, 3])
    assert pm.cp_layout_shape_stride == ((4,), (1,)) and pm.cp_pe_table.dtype == torch.int32
    pm = PeMap.from_mesh_placements(fake_mesh((2, 4)), [Shard(1), Shard(2)], my_rank=5, device=torch.device("cpu"))
    assert (pm.cp, pm.my_cp_rank, pm.cp_axis_sizes, pm.cp_shard_tensor_dims) == (8, 5, (2, 4), (1, 2))
    # dp axis replicated: the cp group holds only this rank's dp slice, in mesh order
    pm = PeMap.from_mesh_placements(fake_mesh((2, 2, 2)), [Replicate(), Shard(1), Shard(2)], my_rank=6,
                                    device=torch.device("cpu"))
    assert pm.cp_pe_table.tolist() == [4, 5, 6, 7] and pm.my_cp_rank == 2 and pm.cp_axes == (1, 2)
    with pytest.raises(ValueError, match="placements length"):
        PeMap.from_mesh_placements(fake_mesh((4,)), [Shard(1), Shard(2)], my_rank=0)
    with pytest.raises(ValueError, match="No sharded mesh axis"):
        PeMap.from_mesh_placements(fake_mesh((4,)), [Replicate()], my_rank=0)
    with pytest.raises(ValueError, match="appears 0 times"):
        PeMap.from_mesh_placements(fake_mesh((4,)), [Shard(1)], my_rank=9)


def test_geometry_from_pe_map_orders_peers_by_row_then_column_block():
    dev = torch.device("cpu")
    g = front._geometry_from_pe_map(PeMap.from_mesh_placements(fake_mesh((2, 4)), [Shard(1), Shard(2)], my_rank=6, device=dev))
    assert (g.cp0, g.cp1, g.rank, g.peers) == (2, 4, 6, tuple(range(8)))
    # columns listed first in the mesh: flat mesh order is (col block, row block); the kernels want the transpose
    g = front._geometry_from_pe_map(PeMap.from_mesh_placements(fake_mesh((4, 2)), [Shard(2), Shard(1)], my_rank=3, device=dev))
    assert (g.cp0, g.cp1) == (2, 4)
    assert g.peers == (0, 2, 4, 6, 1, 3, 5, 7) and g.peers[g.rank] == 3
    g = front._geometry_from_pe_map(PeMap.from_mesh_placements(fake_mesh((4,)), [Shard(2)], my_rank=1, device=dev))
    assert (g.cp0, g.cp1, g.rank) == (1, 4, 1)
    with pytest.raises(ValueError, match="distinct token dim"):
        front._geometry_from_pe_map(PeMap.from_mesh_placements(fake_mesh((2, 2)), [Shard(1), Shard(1)], my_rank=0, device=dev))


# ------------------------------------------------------------------------------------------------
# sharding validation
# ------------------------------------------------------------------------------------------------
def test_validate_trimul_sharding():
    assert validate_trimul_sharding([Shard(0), Shard(1), Shard(2)], 3) == (1, 2)
    assert validate_trimul_sharding([Shard(1)], 1) == (0,)
    with pytest.raises(ValueError, match="feature dim"):
        validate_trimul_sharding([Shard(1), Shard(3)], 2)
    with pytest.raises(ValueError, match="at least one token axis"):
        validate_trimul_sharding([Shard(0)], 1)
    with pytest.raises(ValueError, match="placements length"):
        validate_trimul_sharding([Shard(1)], 2)
    assert _token_split_factor(fake_mesh((2, 4)), [Shard(0), Shard(2)]) == 4
    assert _token_split_factor(fake_mesh((2, 1)), [Shard(0), Shard(1)]) == 1
    assert _rowmaj_stride((2, 3, 4)) == (12, 4, 1)
    assert not _is_dtensor(torch.zeros(1))


def test_effective_placements_uses_real_replicate():
    from torch.distributed.tensor import Replicate as TReplicate, Shard as TShard

    eff = _effective_placements(fake_mesh((1, 4)), [TShard(1), TShard(2)])
    assert isinstance(eff[0], TReplicate) and eff[1] == TShard(2)


# ------------------------------------------------------------------------------------------------
# weights
# ------------------------------------------------------------------------------------------------
def _layer(D=16, bias=False):
    layer = nn.Module()
    layer.norm_in, layer.norm_out = nn.LayerNorm(D), nn.LayerNorm(D)
    layer.p_in, layer.g_in = nn.Linear(D, 2 * D, bias=bias), nn.Linear(D, 2 * D, bias=bias)
    layer.p_out, layer.g_out = nn.Linear(D, D, bias=bias), nn.Linear(D, D, bias=bias)
    return layer


def test_weight_adapters_roundtrip():
    assert len(W_KEYS) == 8 and len(W_PROJ_BIAS_KEYS) == 4
    layer = _layer(bias=True)
    w = weights_from_trimul_module(layer)
    assert set(w) == set(W_KEYS) | set(W_PROJ_BIAS_KEYS)
    assert w["p_in_w"].shape == (32, 16) and not w["p_in_w"].requires_grad and w["p_in_b"] is not None
    w2 = weights_from_trimul_module(trimul_module_from_weights(w))
    for k in w:
        assert torch.equal(w[k], w2[k])
    nob = weights_from_trimul_module(_layer(bias=False), dtype=torch.bfloat16)
    assert all(nob[k] is None for k in W_PROJ_BIAS_KEYS) and nob["p_out_w"].dtype is torch.bfloat16
    broken = _layer()
    del broken.g_out
    with pytest.raises(AttributeError, match="g_out"):
        weights_from_trimul_module(broken)
    with pytest.raises(KeyError):
        trimul_module_from_weights({k: v for k, v in w.items() if k != "p_in_w"})
    with pytest.raises(ValueError):
        trimul_module_from_weights(dict(w, norm_in_b=None))


# ------------------------------------------------------------------------------------------------
# tuning + front door (construction only; no GPU)
# ------------------------------------------------------------------------------------------------
def test_tuning_surface():
    assert TriMulTuning().to_engine_kwargs() == {}
    t = TriMulTuning(front=FrontTuning(tile_mn=(128, 64)), back=BackTuning(cluster_n=2), persistent=True)
    assert t.to_engine_kwargs() == {"front_tile_mn": (128, 64), "back_cluster_n": 2, "is_persistent": True}
    legal = {n for n, p in inspect.signature(front.TriMulAutotuned.__init__).parameters.items()
             if p.kind is inspect.Parameter.KEYWORD_ONLY}
    assert set(t.to_engine_kwargs()) <= legal
    # the engine's keyword-only surface is partitioned: every knob is either reachable through the tuning
    # types or listed in NOT_EXPOSED with a reason (the reference's own test of this module checks the same)
    from fold_cp_ops_b200.distributed.workflows.trimul_tuning import OutGateTuning, TransportTuning
    exposed = set(TriMulTuning._ENGINE_KEYS.values())
    for group in (FrontTuning, BackTuning, OutGateTuning, TransportTuning):
        exposed |= set(group._ENGINE_KEYS.values())
        assert all(getattr(group(), f) is None for f in group.__dataclass_fields__)
    assert exposed | set(NOT_EXPOSED) == legal and not (exposed & set(NOT_EXPOSED))
    # the sm_100a knobs are real: they reach the engine under its own spelling
    real = TriMulTuning(back=BackTuning(contract_form="single"), front=FrontTuning(fixed_order=True),
                        transport=TransportTuning(wait_timeout_ms=500.0))
    assert real.to_engine_kwargs() == {"front_fixed_order": True, "contract_form": "single", "wait_timeout_ms": 500.0}
    assert TriMulTuning(back=BackTuning(band_rows=4, fixed_start=True)).to_engine_kwargs() == {
        "contract_band_rows": 4, "contract_fixed_start": True}
    from fold_cp_ops_b200 import kernels as K
    assert K.make_tuning("pair", contract_band_rows=4).contract_band_rows == 4 and K.make_tuning().contract_band_rows == 0
    with pytest.raises(ValueError, match="contract_band_rows"):
        K.make_tuning(contract_band_rows=-1)
    assert K.make_tuning(contract_pace_ns=-1).contract_pace_ns == -1 and K.make_tuning().contract_pace_ns == 0
    with pytest.raises(ValueError, match="contract_pace_ns"):
        K.make_tuning(contract_pace_ns=200000)
    assert TriMulTuning(back=BackTuning(pace_ns=5000)).to_engine_kwargs() == {"contract_pace_ns": 5000}
    with pytest.raises(TypeError, match="tile_mm"):
        FrontTuning(tile_mm=(128, 128))
    with pytest.raises(Exception):
        FrontTuning().tile_mn = (1, 2)


def test_incoming_store_variant_is_total():
    f = front.incoming_store_variant
    assert [f("outgoing", c) for c in (1, 2, 4)] == ["plain"] * 3
    assert f("incoming", 1) == "composite_k" and f("incoming", 4, 3) == "route2_ni"
    for bad in (dict(direction="sideways", cp1=1), dict(direction="incoming", cp1=0),
                dict(direction="incoming", cp1=1, batch=0)):
        with pytest.raises(ValueError):
            f(**bad)


def test_public_names_and_ctor_validation():
    assert front.__all__ == ["TriangularMultiplication", "trimul_a2a"]
    layer = _layer(128)
    with pytest.raises(ValueError, match="direction"):
        front.TriangularMultiplication(layer, "sideways", None, None)
    with pytest.raises(TypeError, match="DeviceMesh"):
        front.TriangularMultiplication(layer, "outgoing", object(), None)
    with pytest.raises(ValueError, match="placements has"):
        front.TriangularMultiplication(layer, "outgoing", fake_mesh((2,)), None, placements=[Shard(1), Shard(2)])
    with pytest.raises(ValueError, match="3-D mesh"):
        front.TriangularMultiplication(layer, "outgoing", fake_mesh((2, 2, 2)), None)
    with pytest.raises(ValueError, match="feature dim"):
        front.TriangularMultiplication(layer, "outgoing", fake_mesh((2, 2)), SimpleNamespace(rank=0, device=torch.device("cpu")),
                                       placements=[Shard(1), Shard(3)])
    broken = _layer(128)
    del broken.p_out
    with pytest.raises(AttributeError, match="p_out"):
        front.TriangularMultiplication(broken, "outgoing", None, None)
    m = front.TriangularMultiplication(layer, "incoming", None, None)
    assert m.incoming_variant == "cp1_fallback" and m.direction == "incoming"
    for name in ("norm_in", "p_in", "g_in", "norm_out", "p_out", "g_out"):
        assert getattr(m, name) is getattr(layer, name)
    assert all(m._w[k].dtype is torch.float32 for k in ("norm_in_w", "norm_in_b", "norm_out_w", "norm_out_b"))
    with pytest.raises(ValueError):
        m.prepare(n_token=0)
    assert m.prepare(n_token=64) is None
    m.free()
    # cp > 1 module on a fabricated mesh: construction resolves cp and the peer map, allocates nothing
    dm = SimpleNamespace(rank=5, device=torch.device("cpu"))
    m = front.TriangularMultiplication(layer, "incoming", fake_mesh((2, 4)), dm, placements=[Shard(1), Shard(2)])
    assert (m._cp, m._cp_axis_sizes, m._cp1, m.incoming_variant) == (8, (2, 4), 4, "unbuilt")
    m = front.TriangularMultiplication(layer, "incoming", fake_mesh((1, 1)), dm, placements=[Shard(1), Shard(2)])
    assert m._cp == 1


def test_trimul_a2a_rejects_unknown_kwargs_before_anything_else():
    with pytest.raises(TypeError, match="did you mean 'composite_k'"):
        front.trimul_a2a(torch.zeros(1, 8, 8, 128), {}, torch.bfloat16, composite_kk=True)
    with pytest.raises(TypeError, match="DTensor or local Tensor"):
        front.trimul_a2a("x", {}, torch.bfloat16)


# ------------------------------------------------------------------------------------------------
# C ABI
# ------------------------------------------------------------------------------------------------
def test_library_exports_every_declared_symbol():
    import re
    from pathlib import Path

    header = (Path(__file__).resolve().parent.parent / "include" / "trimul_sm100.h").read_text()
    declared = set(re.findall(r"\b(trimul_sm100_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.EXPORTED_SYMBOLS), declared ^ set(_lib.EXPORTED_SYMBOLS)
    lib = ctypes.CDLL(str(_lib.library_path()))
    for sym in declared:
        assert hasattr(lib, sym), sym


@pytest.mark.parametrize("form,tile_rows", [("pair", 256), ("single", 128)])
def test_contraction_tile_walk_is_a_permutation_and_rotates_the_owners(form, tile_rows):
    """`trimul_sm100_contract_walk` evaluates, on the host, the function the contraction kernels use to pick
    their next tile.  Whatever the band height, grid shape, rank and start rule, every tile of a plane is visited
    exactly once; a band is walked column by column; every rank starts in its own block of the result; and
    at any position of the walk the ranks of a 1-D grid are in the row blocks of DIFFERENT owners."""
    from fold_cp_ops_b200 import kernels as K

    for N, cp0, cp1 in ((8, 1, 1), (600, 1, 1), (1280, 1, 1), (4096, 1, 1), (4096, 4, 1), (4096, 2, 4), (1536, 2, 2)):
        for band in (0, 1, 3, 8, 64):
            for rank in range(cp0 * cp1):
                for fixed in (False, True):
                    g = K.make_geom(1, N, 128, "incoming", 1e-5, cp0, cp1, rank)
                    t = K.make_tuning(form, contract_band_rows=band, contract_fixed_start=fixed)
                    (ti, tj), walk = K.contract_walk(g, t)
                    assert (ti, tj) == (-(-N // tile_rows), -(-N // 256))
                    assert sorted(walk) == [(i, j) for i in range(ti) for j in range(tj)], (N, cp0, cp1, band, rank)
                    r0, r1 = rank // cp1, rank % cp1
                    start = (0, 0) if fixed else ((r0 * (N // cp0)) // tile_rows % ti, (r1 * (N // cp1)) // 256 % tj)
                    assert walk[0] == start
                    rows = min(band or 8, ti)
                    assert len({c for _, c in walk[:rows]}) == 1 and len({r for r, _ in walk[:rows]}) == rows
    # a NULL tuning is the library's default: CTA pairs, bands of 8, own-block start
    g = K.make_geom(1, 4096, 256, "outgoing", 1e-5, 8, 1, 3)
    assert K.contract_walk(g) == K.contract_walk(g, K.make_tuning("pair", contract_band_rows=8))
    # the rotation: at every position the eight ranks store into eight different owners' row blocks
    walks = [K.contract_walk(K.make_geom(1, 4096, 256, "outgoing", 1e-5, 8, 1, r), K.make_tuning(form))[1]
             for r in range(8)]
    for pos in range(len(walks[0])):
        owners = {w[pos][0] * tile_rows // 512 for w in walks}
        assert len(owners) == 8, (pos, owners)
    with pytest.raises(Exception, match="contract_band_rows"):
        bad = K.make_tuning(form)
        bad.contract_band_rows = -2
        K.contract_walk(g, bad)


def test_ctypes_mirrors_match_the_header_structs(tmp_path):
    """Every struct of include/trimul_sm100.h, as the C compiler lays it out (field names in order, offsets,
    total size: a small program compiled here against the header prints them), against its ctypes mirror
    in `_lib.py`.  A field added on one side only would shift every later field silently."""
    import re
    import shutil
    import subprocess
    from pathlib import Path

    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    inc = Path(__file__).resolve().parent.parent / "include"
    header = (inc / "trimul_sm100.h").read_text()
    mirrors = {"trimul_caps": _lib.Caps, "trimul_geom": _lib.Geom, "trimul_tuning": _lib.Tuning,
               "trimul_status": _lib.Status, "trimul_plan_desc": _lib.PlanDesc, "trimul_workspace": _lib.Workspace,
               "trimul_reshard_plan": _lib.ReshardPlan}
    structs = dict(re.findall(r"typedef struct (\w+) \{(.*?)\} \w+_t;", header, flags=re.S))
    assert set(structs) == set(mirrors), set(structs) ^ set(mirrors)
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "trimul_sm100.h"', 'int main(void) {']
    fields = {}
    for name, body in structs.items():
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = [re.sub(r"\[.*\]", "", d.split()[-1].lstrip("*")) for d in body.split(";") if d.strip()]
        fields[name] = names
        lines.append(f'  printf("{name} size %zu\\n", sizeof(struct {name}));')
        lines += [f'  printf("{name} {f} %zu\\n", offsetof(struct {name}, {f}));' for f in names]
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(inc), str(src), "-o", str(exe)], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    seen = {}
    for line in filter(None, out):
        name, field, value = line.split()
        seen.setdefault(name, {})[field] = int(value)
    for name, mirror in mirrors.items():
        assert [f for f, _ in mirror._fields_] == fields[name], (name, fields[name])
        assert ctypes.sizeof(mirror) == seen[name]["size"], name
        for f, _ in mirror._fields_:
            assert getattr(mirror, f).offset == seen[name][f], (name, f)


def test_loader_refuses_a_library_built_from_other_sources(monkeypatch):
    """The loader compares the digest compiled into the library with the sources beside it (file times do
    not survive a copy of the tree): the real library matches, a library reporting another digest is stale."""
    from fold_cp_ops_b200 import build

    real = ctypes.CDLL(str(_lib.library_path()))
    assert _lib._stale_reason(real) == ""
    real.trimul_sm100_build_id.restype = ctypes.c_char_p
    assert real.trimul_sm100_build_id().decode() == build.source_digest()

    class Other:
        class trimul_sm100_build_id:  # noqa: N801 - mimics a ctypes function object
            restype = argtypes = None

            def __new__(cls):
                return b"0123456789abcdef0123456789abcdef"

    assert "library build id 0123" in _lib._stale_reason(Other)
    monkeypatch.setenv("CPO_TRIMUL_LIB", str(_lib.library_path()))   # an explicitly chosen library is not second-guessed
    assert _lib._stale_reason(Other) == ""


def test_geometry_refusals_come_back_as_value_errors():
    for kw, pat in ((dict(n=12), "multiple of 8"), (dict(d=64), "not supported"), (dict(d=320), "not supported"), (dict(cp0=3, n=24), "must divide"),
                    (dict(cp0=2, cp1=2, rank=7), "rank"), (dict(cp0=4, cp1=4), "ranks"),
                    (dict(cp0=2, n=24), "multiples of 8")):
        base = dict(batch=1, n=64, d=128, direction="outgoing", eps=1e-5, cp0=1, cp1=1, rank=0)
        base.update(kw)
        with pytest.raises(ValueError, match=pat):
            K.workspace_bytes(K.make_geom(**base))
    assert K.reshard_plan(K.make_geom(1, 64, 384, "outgoing", 1e-5, cp0=8, cp1=1, rank=5)).d_loc == 48   # not a power of two
    ws = K.workspace_bytes(K.make_geom(2, 64, 256, "incoming", 1e-5, cp0=2, cp1=2, rank=3))
    assert ws.ab_bytes == 2 * 64 * 2 * 64 * 64 * 2 and ws.tri_bytes == 256 * 2 * 32 * 32 * 2 == ws.gate_bytes


# ------------------------------------------------------------------------------------------------
# the two reshards, every rank simulated in one process (index arithmetic of the C ABI)
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
@pytest.mark.parametrize("cp0,cp1", [(1, 1), (2, 1), (4, 1), (1, 2), (2, 2), (2, 4)])
def test_reshard_plans_tile_every_buffer_exactly_once(direction, cp0, cp1):
    B, N, D = 2, 32, 128
    cp = cp0 * cp1
    d_loc = D // cp
    # value = unique id of (half, channel, batch, i, j) in the GLOBAL a|b tensor
    hh, cc, bb, ii, jj = np.meshgrid(np.arange(2), np.arange(D), np.arange(B), np.arange(N), np.arange(N), indexing="ij")
    gid = (((hh * D + cc) * B + bb) * N + ii) * N + jj
    ab_bufs = [np.full(2 * d_loc * B * N * N, -1, dtype=np.int64) for _ in range(cp)]
    for r in range(cp):
        p = K.reshard_plan(K.make_geom(B, N, D, direction, 1e-5, cp0, cp1, r))
        ni, nj = N // cp0, N // cp1
        assert (p.ni_loc, p.nj_loc, p.d_loc, p.planes, p.rows) == (ni, nj, d_loc, d_loc * B, B * ni * nj)
        i_off, j_off = (r // cp1) * ni, (r % cp1) * nj
        b, line, w = np.meshgrid(np.arange(B), np.arange(p.n_lines), np.arange(p.n_walk), indexing="ij")
        row = b * p.batch_rows + line * p.line_rows + w * p.walk_rows           # row of the local x block
        assert sorted(row.ravel().tolist()) == list(range(B * ni * nj))          # the walk covers every local token once
        i_l, j_l = (row % (ni * nj)) // nj, row % nj
        tok = p.dst_base + line * p.dst_line + w
        for h in range(2):
            for c in range(D):
                owner, cl = c // d_loc, c % d_loc
                dst = ((h * d_loc + cl) * B + b) * p.plane_elems + tok
                assert (ab_bufs[owner][dst.ravel()] == -1).all()                 # nobody wrote here before
                ab_bufs[owner][dst.ravel()] = gid[h, c, b, i_off + i_l, j_off + j_l].ravel()
    for s in range(cp):
        buf = ab_bufs[s].reshape(2, d_loc, B, N, N)
        assert (buf >= 0).all()                                                  # every element written
        want = gid[:, s * d_loc:(s + 1) * d_loc]                                 # (2, d_loc, B, i, j)
        if direction == "incoming":
            want = want.transpose(0, 1, 2, 4, 3)                                 # plane[row = j][col = i]
        assert (buf == want).all()
    # back reshard: rank s owns channels [s*d_loc, (s+1)*d_loc) of tri over the full grid
    tri_bufs = [np.full(D * B * (N // cp0) * (N // cp1), -1, dtype=np.int64) for _ in range(cp)]
    c_, b_, i_, j_ = np.meshgrid(np.arange(d_loc), np.arange(B), np.arange(N), np.arange(N), indexing="ij")
    for s in range(cp):
        p = K.reshard_plan(K.make_geom(B, N, D, direction, 1e-5, cp0, cp1, s))
        assert p.chan_offset == s * d_loc
        owner = (i_ // p.ni_loc) * cp1 + (j_ // p.nj_loc)
        dst = ((p.chan_offset + c_) * B + b_) * (p.ni_loc * p.nj_loc) + (i_ % p.ni_loc) * p.nj_loc + (j_ % p.nj_loc)
        val = (((p.chan_offset + c_) * B + b_) * N + i_) * N + j_
        for o in range(cp):
            sel = owner == o
            assert (tri_bufs[o][dst[sel]] == -1).all()
            tri_bufs[o][dst[sel]] = val[sel]
    for o in range(cp):
        ni, nj = N // cp0, N // cp1
        buf = tri_bufs[o].reshape(D, B, ni, nj)
        i0, j0 = (o // cp1) * ni, (o % cp1) * nj
        dd, bb2, il, jl = np.meshgrid(np.arange(D), np.arange(B), np.arange(ni), np.arange(nj), indexing="ij")
        assert (buf == ((dd * B + bb2) * N + (i0 + il)) * N + (j0 + jl)).all()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("CPO_TRIMUL_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(_lib.TrimulLibraryError, match="no PyTorch or CPU fallback"):
        _lib.load()


def test_engine_refuses_cpu_device():
    from fold_cp_ops_b200.engine import TriMulEngine

    with pytest.raises(RuntimeError, match="no CPU path"):
        TriMulEngine(weights_from_trimul_module(_layer(128)), device=torch.device("cpu"))
