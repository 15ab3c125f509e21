"""Ahead-of-time build of ``libtrimul_sm100.so`` with nvcc for sm_100a.

The library is built in-tree (next to this file) so that it travels with a snapshot of the
repository; there is no JIT and no torch extension machinery involved.  ``python -m
fold_cp_ops_b200.build`` rebuilds it; :func:`ensure_built` rebuilds only when a source is newer
than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libtrimul_sm100.so"

SOURCES = ("trimul_capi.cu", "ln_gated_proj.cu", "tri_contract.cu", "tri_contract_pair.cu", "ln_out_proj.cu", "peer_sync.cu",
           "forward_static.cu")
HEADERS = ("sm100_ptx.cuh", "trimul_common.cuh", "trimul_kernels.h", "tri_contract_epilogue.cuh")

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
    "--use_fast_math",
    "-diag-suppress", "177",
)


def source_digest() -> str:
    """sha256 over the CUDA sources, their headers and the public header, in a fixed order.  Compiled into
    the library (``trimul_sm100_build_id``) so that the loader can tell a library built from other sources
    without relying on file times, which a copy of the tree does not preserve."""
    import hashlib

    h = hashlib.sha256()
    for f in [CSRC / s for s in SOURCES + HEADERS] + [PKG_DIR.parent / "include" / "trimul_sm100.h"]:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:32]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; libtrimul_sm100.so cannot be built")
    return cand


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [PKG_DIR.parent / "include" / "trimul_sm100.h"]
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False, ptxas_info: bool = False, ablate: int = 0) -> Path:
    """Compile every kernel for sm_100a into one shared library; returns its path.

    ``ablate`` != 0 builds a PROFILING library ``libtrimul_sm100_ablate<bits>.so`` beside the real one, in
    which roles of the projection kernel do no work (``TRIMUL_ABLATE`` in ``csrc/ln_gated_proj.cu``); select
    it with ``CPO_TRIMUL_LIB``.  Its results are wrong by construction; it only exists to be timed."""
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    out = LIB_PATH if not ablate else PKG_DIR / f"libtrimul_sm100_ablate{int(ablate)}.so"
    extra = [f"-DTRIMUL_ABLATE={int(ablate)}"] if ablate else []
    extra.append(f'-DTRIMUL_BUILD_ID="{source_digest()}"')
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if ptxas_info else []), "-o", str(out), *srcs]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose or ptxas_info:
        sys.stderr.write(proc.stderr)
    return out


def ensure_built() -> Path:
    if is_stale():
        build()
    return LIB_PATH


if __name__ == "__main__":
    bits = int(sys.argv[sys.argv.index("--ablate") + 1]) if "--ablate" in sys.argv else 0
    print(build(verbose=True, ptxas_info="--ptxas" in sys.argv, ablate=bits))
