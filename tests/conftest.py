"""pytest configuration: the ``gpu`` marker and import paths.

``-m "not gpu"`` runs everywhere (oracle vs golden vectors, host-side logic, C-ABI symbol check,
gloo multi-process tests); ``-m gpu`` needs a B200 and drives the CUDA kernels through the C ABI.
"""
import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def reference_root():
    """A checkout of the reference project, if one is around: ``REFERENCE_ROOT``, else a directory named
    ``reference`` beside this repository.  ``None`` when there is none (the GPU box has none)."""
    env = os.environ.get("REFERENCE_ROOT")
    cand = Path(env) if env else REPO.parent / "reference"
    return cand if (cand / "fold_cp_ops" / "workflows" / "trimul_autotune.py").exists() else None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x (B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device in this environment")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(REPO / "tests" / "golden" / "trimul_ref_golden.npz")
