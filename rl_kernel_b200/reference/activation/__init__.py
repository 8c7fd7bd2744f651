from rl_kernel_b200.reference.activation.swiglu import NativeSwiGLUOp, swiglu_packed_reference  # noqa: F401
