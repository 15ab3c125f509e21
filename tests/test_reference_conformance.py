"""The reference's own CPU tests of the host layer, run against this package.

The reference project keeps CPU-runnable unit tests for the pieces of the public surface this build
re-implements: the peer map, the layout maps, the sharding validation, the weight adapters and the typed
tuning surface (``tests/distributed/test_{pe_map,layout_map,dtensor_adapter,trimul_weights}.py`` and
``tests/distributed/workflows/test_trimul_tuning.py`` of the reference).  When a checkout of the reference
is available -- ``REFERENCE_ROOT``, or a directory named ``reference`` next to this repository -- they are
executed unmodified in a child process in which the name ``fold_cp_ops`` is this repository's alias package;
only the reference's test-authoring helpers (``fold_cp_ops.testing``, which this build does not ship) are
taken from the checkout.  Without a checkout the test is skipped: nothing here travels with the repository.
"""
import subprocess
import sys

import pytest

from tests.conftest import REPO, reference_root

_BOOT = """
import os, sys
repo, ref = sys.argv[1], sys.argv[2]
sys.dont_write_bytecode = True
sys.path.insert(0, repo)
import fold_cp_ops                                              # this repository's alias package
fold_cp_ops.__path__.append(os.path.join(ref, "fold_cp_ops"))   # fall-through for fold_cp_ops.testing only
import pytest
sys.exit(pytest.main(sys.argv[3:]))
"""

_SUITES = {
    "host_layer": ("tests/distributed/test_pe_map.py", "tests/distributed/test_layout_map.py",
                   "tests/distributed/test_dtensor_adapter.py", "tests/distributed/test_trimul_weights.py"),
    "tuning_surface": ("tests/distributed/workflows/test_trimul_tuning.py",),
}


@pytest.mark.parametrize("suite", sorted(_SUITES))
def test_reference_cpu_tests_pass_against_this_package(suite, tmp_path):
    ref = reference_root()
    if ref is None:
        pytest.skip("no checkout of the reference next to this repository (set REFERENCE_ROOT to run this)")
    files = [str(ref / f) for f in _SUITES[suite]]
    missing = [f for f in files if not (ref / f[len(str(ref)) + 1:]).exists()]
    if missing:
        pytest.skip(f"the reference checkout has no {missing}")
    cmd = [sys.executable, "-c", _BOOT, str(REPO), str(ref), "-q", "-p", "no:cacheprovider", f"--rootdir={tmp_path}",
           "-c", "/dev/null", *files]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=tmp_path, timeout=600)
    tail = (proc.stdout + proc.stderr)[-2500:]
    assert proc.returncode == 0, f"the reference's {suite} tests fail against this package:\n{tail}"
    assert " passed" in proc.stdout and " failed" not in proc.stdout, tail
