from rl_kernel_b200.ops.attention.attention import (AttentionOp, causal_attention, decode_attention,  # noqa: F401
                                                    varlen_tiles)
from rl_kernel_b200.ops.attention.preprocess import AttentionPreprocessor  # noqa: F401
from rl_kernel_b200.ops.attention.projection import AttentionProjectionOp  # noqa: F401
from rl_kernel_b200.ops.attention.paged import PagedKVCache, paged_attention  # noqa: F401
from rl_kernel_b200.ops.attention.prefix_shared import PrefixSharedAttentionOp, prefix_shared_attention  # noqa: F401
