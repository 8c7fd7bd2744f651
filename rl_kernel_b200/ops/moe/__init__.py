from rl_kernel_b200.ops.moe.experts import MoEBuffers, MoEExperts, MoEWeights  # noqa: F401
