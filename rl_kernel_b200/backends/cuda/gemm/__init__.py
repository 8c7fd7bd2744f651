from rl_kernel_b200.backends.cuda.gemm.det_gemm import (DetGemmOp, det_gemm_backend, det_gemm_backend_id,  # noqa: F401
                                                         det_gemm_fallback_reason, det_gemm_linear,
                                                         det_gemm_linear_input_gradient, det_gemm_linear_weight_gradient,
                                                         deterministic_gemm)
