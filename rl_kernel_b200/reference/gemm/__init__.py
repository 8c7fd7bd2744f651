from rl_kernel_b200.reference.gemm.det_gemm import NativeGemmOp, det_gemm_reference  # noqa: F401
