from rl_kernel_b200.reference.packing.pack import NativePackOp, cu_seqlens_from_lengths  # noqa: F401
