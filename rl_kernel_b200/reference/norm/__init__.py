from rl_kernel_b200.reference.norm.rms_norm import NativeRMSNormOp, rms_norm_reference  # noqa: F401
