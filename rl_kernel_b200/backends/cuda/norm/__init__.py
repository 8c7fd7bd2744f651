from rl_kernel_b200.backends.cuda.norm.rmsnorm import RMSNormCuda, RMSNormCudaOp, rmsnorm_cuda  # noqa: F401
