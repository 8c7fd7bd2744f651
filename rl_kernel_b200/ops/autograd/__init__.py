from rl_kernel_b200.ops.autograd.backward_runtime import record_backward, backward_records  # noqa: F401
from rl_kernel_b200.ops.autograd.canonical_backward import CanonicalBackwardSession, active_session  # noqa: F401
from rl_kernel_b200.ops.autograd.vjp_fp32 import rms_norm_vjp_fp32, swiglu_vjp_fp32  # noqa: F401
