from rl_kernel_b200.reference.rope.rope import NativeRoPEOp, qk_norm_rope_reference, rope_tables  # noqa: F401
