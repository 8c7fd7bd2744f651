"""Build hook: ``pip install .`` / ``python setup.py build_ext --inplace`` compiles the sm_100a library in-tree
(``rl_kernel_b200/librlk_b200.so``) with nvcc before the Python packages are collected.  Metadata lives in pyproject.toml."""
from setuptools import setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py


def _build_native() -> None:
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("rlk_csrc_build", Path(__file__).parent / "rl_kernel_b200" / "csrc" / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()


class BuildNative(build_ext):
    def run(self):
        _build_native()


class BuildPyWithNative(build_py):
    def run(self):
        import os

        if os.environ.get("RLK_SKIP_NATIVE_BUILD") != "1":
            _build_native()
        super().run()


setup(cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative})
