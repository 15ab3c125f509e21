"""Generate the golden vectors under tests/golden/ from the REFERENCE's own oracle.

Run where the reference checkout is importable (its path in ``REFERENCE_ROOT``):

    python tests/golden/make_golden.py

For every case listed in ``CASES`` it builds the seeded inputs with
``oracle.trimul_oracle.make_case`` (numpy RandomState stream: identical on every machine), rounds
x and the projection matrices to bf16 exactly as the kernels receive them, evaluates the
reference's ``fold_cp_ops.workflows.trimul_autotune.trimul_ref`` in fp32 on the CPU and stores the
fp32 output (plus a checksum of the inputs) in ``trimul_ref_golden.npz``.  The reference's eager
``nn.Module`` spelling (benchmark/distributed/trimul_dtensor_reference.py:1687-1915) is evaluated
on the first case too and must agree bitwise with ``trimul_ref`` in fp32.
"""
from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from oracle.trimul_oracle import bf16_round_case, make_case, weights_of  # noqa: E402

# name -> make_case kwargs + direction.  Small on purpose: the file stays a few hundred KB.
CASES = {
    "out_n16_d128_plain": dict(B=1, N=16, D=128, seed=101, ln_affine=False, bias="none", mask="none", direction="outgoing"),
    "in_n16_d128_plain": dict(B=1, N=16, D=128, seed=102, ln_affine=False, bias="none", mask="none", direction="incoming"),
    "out_n16_d128_full": dict(B=2, N=16, D=128, seed=103, ln_affine=True, bias="all", mask="random", direction="outgoing"),
    "in_n16_d128_full": dict(B=2, N=16, D=128, seed=104, ln_affine=True, bias="all", mask="pad", direction="incoming"),
    "out_n8_d256_full": dict(B=1, N=8, D=256, seed=105, ln_affine=True, bias="out", mask="ones", direction="outgoing"),
    "in_n8_d256_full": dict(B=1, N=8, D=256, seed=106, ln_affine=True, bias="all", mask="random", direction="incoming"),
}


def input_digest(case) -> str:
    h = hashlib.sha256()
    for k in sorted(case):
        v = case[k]
        h.update(k.encode())
        if v is not None:
            h.update(np.ascontiguousarray(v.numpy()).tobytes())
    return h.hexdigest()


def main() -> None:
    ref_root = os.environ.get("REFERENCE_ROOT")
    if not ref_root:
        raise SystemExit("set REFERENCE_ROOT to a checkout of the reference project (the golden vectors are its outputs)")
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from fold_cp_ops.workflows.trimul_autotune import trimul_ref  # type: ignore

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    out = {}
    for name, kw in CASES.items():
        kw = dict(kw)
        direction = kw.pop("direction")
        case = bf16_round_case(make_case(**kw))
        ref = trimul_ref(case["x"], direction, case["mask"], **weights_of(case), eps=1e-5)
        out[name] = ref.numpy().astype(np.float32)
        out[name + "__digest"] = np.frombuffer(bytes.fromhex(input_digest(case)), dtype=np.uint8)
        print(f"{name}: out {tuple(ref.shape)} max|ref|={ref.abs().max():.4f}")

    # second spelling of the reference oracle: the eager nn.Module (no projection biases; in fp32
    # it must agree bitwise with trimul_ref)
    from benchmark.distributed.trimul_dtensor_reference import (  # type: ignore
        TriangularMultiplicationIncoming,
        TriangularMultiplicationOutgoing,
    )

    for direction, cls in (("outgoing", TriangularMultiplicationOutgoing), ("incoming", TriangularMultiplicationIncoming)):
        case = bf16_round_case(make_case(B=1, N=16, D=128, seed=107, ln_affine=True, bias="none", mask="random"))
        mod = cls(128)
        with torch.no_grad():
            mod.norm_in.weight.copy_(case["norm_in_w"]); mod.norm_in.bias.copy_(case["norm_in_b"])
            mod.norm_out.weight.copy_(case["norm_out_w"]); mod.norm_out.bias.copy_(case["norm_out_b"])
            for nm in ("p_in", "g_in", "p_out", "g_out"):
                getattr(mod, nm).weight.copy_(case[nm + "_w"])
            eager = mod(case["x"], case["mask"])
        ref = trimul_ref(case["x"], direction, case["mask"], **weights_of(case), eps=1e-5)
        diff = (eager - ref).abs().max().item()
        print(f"eager module vs trimul_ref ({direction}): max|diff| = {diff}")
        assert diff == 0.0, "the two reference spellings disagree"
        out[f"eager_{direction}_n16_d128"] = eager.numpy().astype(np.float32)
    np.savez_compressed(HERE / "trimul_ref_golden.npz", **out)
    print("wrote", HERE / "trimul_ref_golden.npz")


if __name__ == "__main__":
    main()
