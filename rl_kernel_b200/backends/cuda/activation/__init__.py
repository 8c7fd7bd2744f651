from rl_kernel_b200.backends.cuda.activation.swiglu import SiLUCudaOp, SwiGLUCudaOp  # noqa: F401
