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

from rl_engine._legacy import LEGACY_ALIASES

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


class _NamespaceLoader(importlib.abc.Loader):
    """An empty package for a legacy path that only exists as a prefix of other legacy paths
    (``rl_engine.kernels``, ``rl_engine.kernels.ops`` ...)."""

    def create_module(self, spec):
        return None

    def exec_module(self, module):
        module.__path__ = []


_LEGACY_PACKAGES = {".".join(k.split(".")[:i]) for k in LEGACY_ALIASES for i in range(1, len(k.split(".")))}


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        rel = fullname[len(_PREFIX):]
        if rel == "_legacy":
            return None                                   # a real file of this package
        legacy_parent = rel in _LEGACY_PACKAGES and rel not in LEGACY_ALIASES
        rel = LEGACY_ALIASES.get(rel, rel)                # old path -> canonical path (same module object)
        real = _TARGET + rel
        try:
            real_spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            real_spec = None
        if real_spec is None:
            if legacy_parent:
                return importlib.util.spec_from_loader(fullname, _NamespaceLoader(), is_package=True)
            return None
        spec = importlib.util.spec_from_loader(fullname, _AliasLoader(real),
                                               is_package=real_spec.submodule_search_locations is not None)
        return spec


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

__version__ = _impl.__version__
# ``_legacy`` is the one real file here; every other sub-module is resolved by the alias finder


def __getattr__(name):
    return getattr(_impl, name)
