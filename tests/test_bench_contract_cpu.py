"""The reference arm of bench.py runs on the host cores alone and prints one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _run(extra_env=None):
    env = dict(os.environ)
    env.pop("RANK", None)
    env.update(extra_env or {})
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    return p.stdout.strip().splitlines()


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    lines = _run()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "trimul_fwd_tflops" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "readme_n4096_d256"
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and "N=" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_is_silent_on_other_ranks():
    assert _run({"RANK": "1", "WORLD_SIZE": "2"}) == []


def test_spot_check_patch_oracle_agrees_with_the_full_oracle():
    """bench.py's full-size parity check evaluates the oracle on a patch only (rows / columns of the input
    it needs).  On a small case its patch must agree with the full CPU oracle, for both directions and with
    the padding mask, and it must notice a wrong output element."""
    import torch

    import bench
    from oracle.trimul_oracle import trimul_oracle

    wl = dict(B=2, N=160, D=128, mask="pad")
    dev = torch.device("cpu")
    w = bench.make_layer_weights(wl["D"], 0, dev)
    x = torch.randn(wl["B"], wl["N"], wl["N"], wl["D"], generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    tm = bench.token_mask(wl["mask"], wl["N"])
    mask = (tm[:, None] * tm[None, :]).expand(wl["B"], -1, -1)
    for direction in ("outgoing", "incoming"):
        full = trimul_oracle(x.float(), direction, mask, **{k: (None if v is None else v.float()) for k, v in w.items()})
        res = bench.spot_check(w, x, full, wl, direction, 1, 1, 1, 0, 0, 0, dev, rows=2, cols=16)
        assert res["within_bound_on_every_rank"] and res["max_abs_err"] < 1e-3, res
        wrong = full.clone()
        wrong[wl["B"] - 1] += 1.0
        assert not bench.spot_check(w, x, wrong, wl, direction, 1, 1, 1, 0, 0, 0, dev, rows=2, cols=16)["within_bound_on_every_rank"]
