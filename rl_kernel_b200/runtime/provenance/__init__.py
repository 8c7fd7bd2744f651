from rl_kernel_b200.runtime.provenance.identity import code_fingerprint, stable_operator_path  # noqa: F401
