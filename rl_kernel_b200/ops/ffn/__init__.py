from rl_kernel_b200.ops.ffn.qwen3 import Qwen3FFNOp, qwen3_ffn  # noqa: F401
