from rl_kernel_b200.reference.attention.standard_attn import NativeAttentionOp  # noqa: F401
from rl_kernel_b200.reference.attention.blockwise import (  # noqa: F401
    DeterministicCPAttentionReferenceOp, blockwise_attention_reference, merge_two_states)
from rl_kernel_b200.reference.attention.kv_cache import NativeKVCacheAttnOp, StatefulKVCache  # noqa: F401
from rl_kernel_b200.reference.attention.paged_kv import PagedKVReference  # noqa: F401
