"""Context-parallel parity on 2+ GPUs: one process per GPU, NCCL process group, DTensor in/out.

The oracle is evaluated from the GLOBAL fp32 input on the CPU; every rank compares its own shard
with the per-element bound of the reference's distributed gate (``2e-2 + 6e-2 |ref|``,
tests/distributed/workflows/test_trimul_autotuned.py:556 of the reference).  Meshes: 1-D over all
ranks and every 2-D factorisation; both directions; mask / bias / batch variants; repeated
forwards (the flag counters and WAR guards are exercised by running each engine several times).
"""
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

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    os.environ.pop("TORCHELASTIC_RUN_ID", None)
    if str(REPO) not in sys.path:
        sys.path.insert(0, str(REPO))
    try:
        q.put((rank, "ok", _cp_parity(rank, world)))
    except BaseException as exc:  # noqa: BLE001
        q.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()}"))


def _factorisations(world):
    out = [None]
    for a in range(2, world):
        if world % a == 0:
            out.append((a, world // a))
    return out


def _cp_parity(rank, world):
    from torch.distributed.tensor import DTensor, Shard

    from fold_cp_ops_b200.distributed import DistributedManager
    from fold_cp_ops_b200.distributed.trimul_weights import trimul_module_from_weights
    from fold_cp_ops_b200.distributed.workflows.trimul_autotuned import TriangularMultiplication
    from oracle.trimul_oracle import bf16_round_case, make_case, tolerance_bound, trimul_oracle, weights_of

    DistributedManager.initialize(device_type="cuda")
    DistributedManager.init_nvshmem()
    dm = DistributedManager()
    assert dm.nvshmem_initialized and dm.world_size == world
    report = []
    for grid in _factorisations(world):
        DistributedManager.reset_grid_groups()
        DistributedManager.create_grid_group(OrderedDict(cp=grid or world))
        mesh = dm.device_mesh_subgroups if grid else dm.device_mesh
        placements = [Shard(i + 1) for i in range(mesh.ndim)]
        cp0 = int(mesh.shape[0])
        cp1 = int(mesh.shape[1]) if mesh.ndim > 1 else 1
        coord = mesh.get_coordinate()
        r0, r1 = coord[0], (coord[1] if mesh.ndim > 1 else 0)
        for direction in ("outgoing", "incoming"):
            for (B, N, D, bias, mask) in ((1, 64 * max(cp0, cp1), 128, "all", "random"), (2, 128, 256, "none", "pad"),
                                          (1, 128, 384, "all", "pad")):   # wide rows; D / cp is not a power of two
                if D % world or (D // world) % 16 or N % cp0 or N % cp1 or (N // cp0) % 8 or (N // cp1) % 8:
                    continue
                case = bf16_round_case(make_case(B, N, D, seed=20260821 + N + D, bias=bias, mask=mask))
                ref = trimul_oracle(case["x"], direction, case["mask"], **weights_of(case))
                layer = trimul_module_from_weights({k: (None if v is None else v.to(dm.device))
                                                    for k, v in weights_of(case).items()})
                tm = TriangularMultiplication(layer, direction, mesh, dm, placements=placements)
                ni, nj = N // cp0, N // cp1
                sl = (slice(None), slice(r0 * ni, (r0 + 1) * ni), slice(r1 * nj, (r1 + 1) * nj))
                x_loc = case["x"][sl].to(dm.device).bfloat16().contiguous()
                m_loc = case["mask"][sl].to(dm.device).contiguous()
                rowmaj = lambda sh: torch.empty(sh, device="meta").stride()
                x = DTensor.from_local(x_loc, mesh, placements, shape=torch.Size((B, N, N, D)), stride=rowmaj((B, N, N, D)),
                                       run_check=False)
                m = DTensor.from_local(m_loc, mesh, placements, shape=torch.Size((B, N, N)), stride=rowmaj((B, N, N)),
                                       run_check=False)
                for rep in range(3):  # repeated forwards exercise the counters and the WAR guards
                    out = tm(x, m)
                tm.check()  # synchronises; raises DeviceWaitTimeout if any bounded wait expired
                # measured forward: kernel windows, cross-rank wait times and bytes pushed to peers
                tm.collect_stats(True)
                out_stats = tm(x, m)
                st = tm.last_forward_stats()
                tm.collect_stats(False)
                assert torch.equal(out_stats.to_local(), out.to_local())
                assert set(st["wait_ms"]) == {"front", "back", "consumed"} and all(v is not None and v >= 0 for v in st["wait_ms"].values())
                assert all(v > 0 for v in st["stage_ms"].values())
                s_bytes = B * (N // cp0) * (N // cp1) * D * 2
                assert st["bytes_to_peers"] == {"front": 2 * s_bytes * (world - 1) // world, "back": s_bytes * (world - 1) // world}
                # the functional front door builds its own engine (own symmetric buffers) and must agree bit for bit
                from fold_cp_ops_b200.distributed.workflows.trimul_autotuned import trimul_a2a
                cache = {}
                w_dev = {k: (None if v is None else v.to(dm.device)) for k, v in weights_of(case).items()}
                out_fn = trimul_a2a(x, w_dev, torch.bfloat16, direction=direction, mask=m, distributed_manager=dm, _cache=cache)
                torch.cuda.synchronize()
                assert out_fn.placements == x.placements and torch.equal(out_fn.to_local(), out.to_local())
                for eng in cache.values():
                    eng.check()
                    eng.free()
                assert out.shape == x.shape and out.placements == x.placements
                got = out.to_local().float().cpu()
                want = ref[sl]
                err = (got - want).abs()
                bad = int((err > tolerance_bound(want)).sum())
                assert not torch.isnan(got).any()
                assert bad == 0, (f"grid={grid} {direction} B{B} N{N} D{D}: {bad} elements beyond 2e-2+6e-2|ref|, "
                                  f"max|err|={err.max().item():.4f}")
                assert tm.incoming_variant == ("plain" if direction == "outgoing" else
                                               ("composite_k" if mesh.ndim == 1 else "route2_ni"))
                report.append((str(grid), direction, N, D, round(err.max().item(), 4)))
                tm.free()
                torch.distributed.barrier()
    DistributedManager.cleanup()
    return report


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_cp_parity_on_all_visible_gpus():
    world = min(_ngpu(), 8)
    while world > 1 and (128 % world):
        world -= 1
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    deadline = time.time() + 600
    while len(out) < world and time.time() < deadline:
        try:
            rank, status, res = q.get(timeout=1.0)
            out[rank] = (status, res)
        except Exception:
            if not any(p.is_alive() for p in procs) and q.empty():
                break
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
    assert len(out) == world, f"only ranks {sorted(out)} of {world} reported"
    for rank, (status, res) in sorted(out.items()):
        assert status == "ok", f"rank {rank}: {res}"
    print(out[0][1])
