"""``rl_engine`` is the import name RL-Kernel users know; here it is an alias of
``rl_kernel_b200``: ``rl_engine.X.Y`` and ``rl_kernel_b200.X.Y`` are the same module object
(the reference does the same for its legacy alias packages,
docs/architecture/repository-layout.md:143-153).
"""
import importlib
import importlib.abc
import importlib.util
import sys

import rl_kernel_b200 as _impl

_PREFIX = __name__ + "."
_TARGET = _impl.__name__ + "."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, real_name):
        self._real_name = real_name

    def create_module(self, spec):
        return importlib.import_module(self._real_name)

    def exec_module(self, module):
        # the module object is the already-imported implementation module
        sys.modules[_PREFIX + self._real_name[len(_TARGET):]] = module


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        real = _TARGET + fullname[len(_PREFIX):]
        try:
            real_spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real),
                                               is_package=real_spec.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__version__ = _impl.__version__
__path__ = []  # sub-modules are resolved by the alias finder only


def __getattr__(name):
    return getattr(_impl, name)
