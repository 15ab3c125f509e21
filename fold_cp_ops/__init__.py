"""Alias package: ``fold_cp_ops.*`` resolves to ``fold_cp_ops_b200.*``.

Lets code written against the reference package's import paths (for example
``from fold_cp_ops.distributed import DistributedManager`` and
``from fold_cp_ops.distributed.workflows.trimul_autotuned import TriangularMultiplication``)
run on the B200 build unchanged.  Nothing is defined here; a meta-path finder maps every
``fold_cp_ops.x.y`` import to the module object of ``fold_cp_ops_b200.x.y``.
"""
import importlib
import importlib.abc
import importlib.util
import sys

_REAL = "fold_cp_ops_b200"
_ALIAS = __name__


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, real_name):
        self._real_name = real_name

    def create_module(self, spec):
        return importlib.import_module(self._real_name)

    def exec_module(self, module):  # the real module is already initialised
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        real_name = _REAL + fullname[len(_ALIAS):]
        try:
            real_spec = importlib.util.find_spec(real_name)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real_name),
                                               is_package=real_spec.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

from fold_cp_ops_b200 import __version__  # noqa: E402,F401
