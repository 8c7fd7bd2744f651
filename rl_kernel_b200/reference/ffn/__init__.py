from rl_kernel_b200.reference.ffn.ffn import NativeQwen3FFNOp, qwen3_ffn_reference  # noqa: F401
