"""Varlen packing (compaction by mask, cu_seqlens); pure index ops, identical on every device."""
from rl_kernel_b200.reference.packing.pack import NativePackOp as PackOp, cu_seqlens_from_lengths  # noqa: F401
