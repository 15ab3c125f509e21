"""The eager PyTorch + collective comparison baseline computes the same function as the oracle
(checked here in fp32 on CPU, one rank and two gloo ranks)."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from baseline.nccl_cp_trimul import NcclCpTriMul  # noqa: E402
from oracle.trimul_oracle import make_case, trimul_oracle, weights_of  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_single_rank_matches_oracle(direction):
    case = make_case(1, 24, 128, seed=5, bias="all", mask="random")
    ref = trimul_oracle(case["x"], direction, case["mask"], **weights_of(case))
    got = NcclCpTriMul(weights_of(case), dtype=torch.float32).forward(case["x"], direction, case["mask"])
    assert torch.allclose(got, ref, atol=2e-4, rtol=2e-4)


def _worker(rank, world, port, direction, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = make_case(2, 16, 128, seed=9, bias="out", mask="random")
        ref = trimul_oracle(case["x"], direction, case["mask"], **weights_of(case))
        ni = 16 // world
        rows = slice(rank * ni, (rank + 1) * ni)
        got = NcclCpTriMul(weights_of(case), dtype=torch.float32).forward(
            case["x"][:, rows].contiguous(), direction, case["mask"][:, rows].contiguous())
        q.put((rank, bool(torch.allclose(got, ref[:, rows], atol=2e-4, rtol=2e-4))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_two_gloo_ranks_match_oracle(direction):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, direction, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    res = dict(q.get(timeout=5) for _ in range(2))
    assert res == {0: True, 1: True}
