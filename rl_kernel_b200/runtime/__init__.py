"""Runtime dispatch, policy and provenance (parity: rl_engine/runtime).  One backend exists, so the
registry is a strict name -> {b200 kernel, reference} map that records what actually ran."""
from rl_kernel_b200.runtime.policy import RLKernelMode, current_mode, strict_contract_enabled  # noqa: F401
from rl_kernel_b200.runtime.registry import KernelRegistry, OpBackend, kernel_registry, resolve_logp_op_type  # noqa: F401
