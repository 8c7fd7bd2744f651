from rl_kernel_b200.ops.gemm.det_gemm import (DetGemmOp, det_gemm, det_gemm_da, det_gemm_db,  # noqa: F401
                                             det_gemm_fwd, det_gemm_fwd_fp32, det_gemm_linear)
from rl_kernel_b200.ops.gemm.canonical_linear import canonical_linear_fp32  # noqa: F401
