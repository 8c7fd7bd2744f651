"""rl_kernel_b200 — deterministic RL post-training operators written for NVIDIA B200 (sm_100a).

The package keeps the public surface of RL-Kernel's ``rl_engine`` (operator contracts,
registry, reference ops, Qwen3 dense model, weight-sync bridge, integrations, validation,
CLI) on ONE backend: hand-written CUDA for sm_100a in ``librlk_b200.so`` plus PyTorch for the
framework layer.  ``import rl_engine`` resolves to this package (see ``rl_engine/__init__.py``),
so ``rl_engine.runtime.registry.kernel_registry`` and friends keep working.

Sub-packages: ``ops`` (operator entry points), ``reference`` (fp32 PyTorch definitions),
``models``, ``parallel``/``distributed`` (fixed-order collectives and fused
compute+collective ops), ``runtime`` (registry, policy, provenance), ``contracts``,
``integrations``, ``validation``, ``entrypoints``, ``utils``.
"""
import torch  # noqa: F401  (loaded first so CUDA libraries resolve before the native library)

__version__ = "0.1.0"

from rl_kernel_b200.utils.logger import init_logger  # noqa: E402

__all__ = ["__version__", "init_logger"]
