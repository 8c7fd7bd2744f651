from rl_kernel_b200.backends.cuda.rope.rope import RoPESM90Op, RoPESM100Op  # noqa: F401
