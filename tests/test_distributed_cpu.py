"""Multi-process host logic on CPU ranks (gloo, world size 2): the manager's bring-up and meshes,
the peer map on a real DeviceMesh, the front door's construction on a cp=2 mesh, and the
group-uniform guards -- including their failure paths, which are made on the host (a rank that
raises, a rank that never joins a barrier) and never on a GPU."""
import os
import socket
import sys
import time
import traceback
from collections import OrderedDict
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

REPO = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    os.environ.pop("TORCHELASTIC_RUN_ID", None)
    if str(REPO) not in sys.path:
        sys.path.insert(0, str(REPO))
    try:
        res = globals()[fn_name](rank, world)
        q.put((rank, "ok", res))
    except BaseException as exc:  # noqa: BLE001 - reported to the parent
        q.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))


def _run(fn_name, world=2, timeout=120):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    deadline = time.time() + timeout
    while len(out) < world and time.time() < deadline:
        try:
            rank, status, res = q.get(timeout=1.0)
            out[rank] = (status, res)
        except Exception:
            if not any(p.is_alive() for p in procs) and q.empty():
                break
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
    assert len(out) == world, f"only {sorted(out)} of {world} ranks reported"
    for rank, (status, res) in out.items():
        assert status == "ok", f"rank {rank}: {res}"
    return {r: v[1] for r, v in out.items()}


# ------------------------------------------------------------------------------------------------
def _manager_and_meshes(rank, world):
    from torch.distributed.tensor import Shard

    from fold_cp_ops_b200.distributed import DistributedManager, PeMap
    from fold_cp_ops_b200.distributed.workflows.trimul_autotuned import TriangularMultiplication, _geometry_from_pe_map
    import torch.nn as nn

    assert not DistributedManager.is_initialized()
    try:
        DistributedManager()
        raise AssertionError("instantiation before initialize() must raise")
    except RuntimeError as exc:
        assert "before" in str(exc)
    DistributedManager.initialize(device_type="cpu")
    dm = DistributedManager()
    assert (dm.rank, dm.world_size, dm.local_rank, dm.backend, dm.method_init) == (rank, world, rank, "gloo", "ENV")
    assert dm.device == torch.device("cpu") and dm.group_ranks["world"] == list(range(world))
    import warnings

    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        DistributedManager.initialize(device_type="cpu")  # second call: warns, changes nothing
    assert any("already initialized" in str(w.message) for w in caught)
    # symmetric memory needs CUDA devices; on CPU ranks the bring-up refuses with a clear sentence
    try:
        DistributedManager.init_nvshmem()
        raise AssertionError("init_nvshmem on CPU ranks must raise")
    except RuntimeError as exc:
        assert "CUDA" in str(exc)
    # 1-D mesh
    DistributedManager.create_grid_group(OrderedDict(cp=world))
    assert tuple(dm.device_mesh.shape) == (world,) and not dm.has_subgroups
    assert dm.group_ranks["cp"] == list(range(world)) and dm.group_rank["cp"] == rank
    pm = PeMap.from_mesh_placements(dm.device_mesh, [Shard(1)], distributed_manager=dm)
    assert (pm.cp, pm.my_cp_rank, pm.cp_pe_table.tolist()) == (world, rank, list(range(world)))
    geo = _geometry_from_pe_map(pm)
    assert (geo.cp0, geo.cp1, geo.rank) == (world, 1, rank)
    # the front door on a live cp=2 mesh: construction resolves everything and allocates nothing
    D = 128
    torch.manual_seed(0)
    layer = nn.Module()
    layer.norm_in, layer.norm_out = nn.LayerNorm(D), nn.LayerNorm(D)
    layer.p_in, layer.g_in = nn.Linear(D, 2 * D, bias=False), nn.Linear(D, 2 * D, bias=False)
    layer.p_out, layer.g_out = nn.Linear(D, D, bias=False), nn.Linear(D, D, bias=False)
    tm = TriangularMultiplication(layer, "incoming", dm.device_mesh, dm)
    assert (tm._cp, tm._cp_axis_sizes, tm.incoming_variant) == (world, (world,), "unbuilt")
    # factored mesh on the same process group
    DistributedManager.reset_grid_groups()
    assert set(dm.group) == {"world"} and dm.device_mesh is None
    DistributedManager.create_grid_group(OrderedDict(cp=(1, world)))
    assert dm.has_subgroups and tuple(dm.device_mesh.shape) == (world,)
    assert tuple(dm.device_mesh_subgroups.shape) == (1, world)
    assert set(dm.group) >= {"world", "cp", "cp_axis_0", "cp_axis_1"}
    assert dm.subgroups_ranks["cp"] == [[rank], list(range(world))]
    pm2 = PeMap.from_mesh_placements(dm.device_mesh_subgroups, [Shard(1), Shard(2)], distributed_manager=dm)
    assert pm2.cp_axis_sizes == (1, world) and pm2.my_cp_rank == rank
    tm2 = TriangularMultiplication(layer, "outgoing", dm.device_mesh_subgroups, dm)
    # the size-1 row axis is dropped, so the peer map is 1-D over the column axis ...
    assert tm2._cp == world and tm2._cp_axis_sizes == (world,)
    # ... and the kernels' geometry knows it is the COLUMNS that are split
    geo2 = _geometry_from_pe_map(tm2._pe_map)
    assert (geo2.cp0, geo2.cp1, geo2.rank) == (1, world, rank)
    try:
        DistributedManager.create_grid_group(OrderedDict(cp=world + 1))
        raise AssertionError("a mesh that does not multiply to world_size must raise")
    except RuntimeError as exc:
        assert "does not match" in str(exc)
    DistributedManager.cleanup()
    assert not DistributedManager.is_initialized() and not torch.distributed.is_initialized()
    DistributedManager.cleanup()  # idempotent
    return True


def test_manager_meshes_and_front_door_on_two_cpu_ranks():
    _run("_manager_and_meshes")


# ------------------------------------------------------------------------------------------------
def _gate_paths(rank, world):
    import torch.distributed as dist

    from fold_cp_ops_b200.distributed import (BarrierTimeout, CollectiveFailure, CollectiveGate, DistributedManager,
                                              PeerFailure)

    try:
        CollectiveGate()
        raise AssertionError("a gate before init_process_group must raise")
    except RuntimeError as exc:
        assert "initialized" in str(exc)
    DistributedManager.initialize(device_type="cpu")
    gate = CollectiveGate(timeout_s=20)
    assert (gate.rank, gate.world_size) == (rank, world)
    assert gate.agree_bool(rank == 0, op="any") is True
    assert gate.agree_bool(rank == 0, op="all") is False
    assert gate.agree_bool(True, op="all") is True
    try:
        gate.agree_bool(True, op="most")
        raise AssertionError
    except ValueError:
        pass
    # a failure on ONE rank surfaces on EVERY rank, after the reduction
    try:
        with gate.guard("build"):
            if rank == 1:
                raise KeyError("boom")
        raise AssertionError("guard must raise on every rank")
    except CollectiveFailure as exc:
        assert rank == 1 and isinstance(exc.__cause__, KeyError)
    except PeerFailure:
        assert rank == 0
    with gate.guard("fine"):
        pass
    assert gate.should_skip("no nvlink" if rank == 0 else None) is not None
    assert gate.should_skip(None) is None
    gate.barrier()
    try:
        gate.barrier(timeout_s=0)
        raise AssertionError
    except ValueError:
        pass
    # a rank that never joins: the others get BarrierTimeout instead of waiting forever
    outcome = "joined"
    if rank == 0:
        try:
            gate.barrier(timeout_s=1.0)
        except BarrierTimeout:
            outcome = "timeout"
    else:
        time.sleep(2.5)  # arrives after rank 0 gave up
        outcome = "late"
    # the group is desynchronised on purpose now: no further collective; tear down without a barrier
    DistributedManager._state["_group_broken"] = True
    DistributedManager.cleanup()
    return outcome


def test_collective_gate_paths_on_two_cpu_ranks():
    res = _run("_gate_paths")
    assert res[0] == "timeout" and res[1] == "late"


def _oom_vote(rank, world):
    """Rank 1 pretends to have no free device memory: BOTH ranks must refuse the symmetric allocation with
    ``torch.cuda.OutOfMemoryError`` (so neither enters the collective allocation alone); when both have
    room, nobody raises."""
    import torch.distributed as dist

    from fold_cp_ops_b200.distributed import symmetric

    dist.init_process_group("gloo", rank=rank, world_size=world)
    cpu = torch.device("cpu")
    real = torch.cuda.mem_get_info
    outcomes = []
    try:
        for free_by_rank in ({0: 64 << 30, 1: 1 << 20}, {0: 64 << 30, 1: 64 << 30}):
            torch.cuda.mem_get_info = lambda device=None, _f=free_by_rank[rank]: (_f, 180 << 30)
            try:
                symmetric.refuse_unsatisfiable_request(8 << 30, cpu, dist.group.WORLD)
                outcomes.append("fits")
            except torch.cuda.OutOfMemoryError as exc:
                assert "refused on every rank" in str(exc)
                outcomes.append("refused")
    finally:
        torch.cuda.mem_get_info = real
    dist.barrier()
    dist.destroy_process_group()
    return outcomes


def test_symmetric_oom_is_refused_on_every_rank_together():
    res = _run("_oom_vote")
    assert res[0] == ["refused", "fits"] and res[1] == ["refused", "fits"]


# ------------------------------------------------------------------------------------------------
# launcher detection (single process, monkeypatched environment)
# ------------------------------------------------------------------------------------------------
def _clear(monkeypatch):
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "SLURM_PROCID",
              "SLURM_NTASKS", "SLURM_NPROCS", "TORCHELASTIC_RUN_ID", "CPO_DISTRIBUTED_INIT_METHOD"):
        monkeypatch.delenv(k, raising=False)


def test_launcher_detection(monkeypatch):
    from fold_cp_ops_b200.distributed import DistributedManager as DM

    _clear(monkeypatch)
    assert DM._detect_launcher() is None
    monkeypatch.setenv("SLURM_PROCID", "3")
    monkeypatch.setenv("SLURM_NTASKS", "8")
    assert DM._detect_launcher() == "SLURM"
    monkeypatch.setenv("TORCHELASTIC_RUN_ID", "x")  # torchrun inside an srun step: torchrun wins
    assert DM._detect_launcher() == "ENV"
    _clear(monkeypatch)
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    assert DM._detect_launcher() == "ENV"


def test_initialize_refusals(monkeypatch):
    from fold_cp_ops_b200.distributed import DistributedManager as DM

    _clear(monkeypatch)
    assert not DM.is_initialized()
    with pytest.raises(RuntimeError, match="found no launcher environment"):
        DM.initialize(device_type="cpu")
    monkeypatch.setenv("CPO_DISTRIBUTED_INIT_METHOD", "MPI")
    with pytest.raises(ValueError, match="Unknown value"):
        DM.initialize(device_type="cpu")
    monkeypatch.setenv("CPO_DISTRIBUTED_INIT_METHOD", "ENV")
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    with pytest.raises(RuntimeError, match="LOCAL_RANK"):
        DM.initialize(device_type="cpu")
    with pytest.raises(RuntimeError, match="initialize"):
        DM.init_nvshmem()
    with pytest.raises(RuntimeError, match="initialized manager"):
        DM.create_grid_group(OrderedDict(cp=1))
    assert not DM.is_initialized()
    with pytest.raises(RuntimeError, match="CUDA device"):
        DM.symmetric_mempool("cpu")


def test_slurm_first_host():
    from fold_cp_ops_b200.distributed import DistributedManager as DM

    assert DM._slurm_first_host("node[03-05,9],gpu7") == "node03"
    assert DM._slurm_first_host("gpu7,gpu8") == "gpu7"
    assert DM._slurm_first_host("dgx[1,2]") == "dgx1"
    assert DM._slurm_first_host("") is None


# ------------------------------------------------------------------------------------------------
def _spot_check_ranks_1d(rank, world):
    return _spot_check_ranks(rank, world, two_d=False)


def _spot_check_ranks_2d(rank, world):
    return _spot_check_ranks(rank, world, two_d=True)


def _spot_check_ranks(rank, world, two_d):
    """bench.py's full-size parity check on `world` CPU ranks: every rank holds its block of a small global
    tensor and of the full oracle's output; the patch oracle, fed by the line gather, must agree on every
    rank, and a corrupted block on ONE rank must fail the line for everybody."""
    import torch.distributed as dist

    import bench
    from oracle.trimul_oracle import trimul_oracle

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cp0, cp1 = (2, world // 2) if two_d else (world, 1)
        r0, r1 = (rank // cp1, rank % cp1) if two_d else (rank, 0)
        wl = dict(B=1, N=16 * max(cp0, cp1), D=128, mask="pad")
        B, N, D = wl["B"], wl["N"], wl["D"]
        dev = torch.device("cpu")
        w = bench.make_layer_weights(D, 0, dev)
        x = torch.randn(B, N, N, D, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
        tm = bench.token_mask(wl["mask"], N)
        mask = (tm[:, None] * tm[None, :]).expand(B, -1, -1)
        ni, nj = N // cp0, N // cp1
        blk = lambda t: t[:, r0 * ni:(r0 + 1) * ni, r1 * nj:(r1 + 1) * nj].contiguous()
        results = {}
        for direction in ("outgoing", "incoming"):
            full = trimul_oracle(x.float(), direction, mask, **{k: (None if v is None else v.float()) for k, v in w.items()})
            good = bench.spot_check(w, blk(x), blk(full), wl, direction, world, cp0, cp1, rank, r0, r1, dev, rows=2, cols=16)
            assert good["within_bound_on_every_rank"] and good["max_abs_err"] < 1e-3 and good["ranks_checked"] == world, good
            wrong = blk(full).clone()
            if rank == world - 1:
                wrong += 1.0
            bad = bench.spot_check(w, blk(x), wrong, wl, direction, world, cp0, cp1, rank, r0, r1, dev, rows=2, cols=16)
            assert not bad["within_bound_on_every_rank"], bad
            results[direction] = good["max_abs_err"]
        return results
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,grid", [(2, "1d"), (4, "2d"), (8, "1d"), (8, "2d")])
def test_bench_spot_check_gathers_lines_across_ranks(world, grid):
    """Rows over 2 and 8 ranks and the 2-D grids (2,2) and (2,4): the grids `bench.py --gpus N` runs."""
    _run(f"_spot_check_ranks_{grid}", world=world, timeout=300)
