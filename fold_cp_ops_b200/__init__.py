"""fold_cp_ops_b200 -- the context-parallel triangle multiplicative update (TriMul) forward on B200.

Hand-written sm_100a kernels (tcgen05 / TMEM / TMA) behind a C ABI, with the host-side surface of
NVIDIA-BioNeMo/fold-cp-ops for that one path:

    fold_cp_ops_b200.distributed.DistributedManager
    fold_cp_ops_b200.distributed.workflows.trimul_autotuned.{TriangularMultiplication, trimul_a2a}
    fold_cp_ops_b200.workflows.trimul_autotune.trimul_autotuned          (single GPU)

The same modules are importable under the reference's own package name ``fold_cp_ops`` (an alias
package at the repository root), so code written against the reference runs unchanged.
There are no top-level re-exports: import from the defining module.
"""
from ._version import __version__  # noqa: F401
