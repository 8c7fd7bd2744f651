from rl_kernel_b200.reference.logprob.logp import NativeLogpOp  # noqa: F401
from rl_kernel_b200.reference.logprob.tile_logp import (  # noqa: F401
    NativeBatchInvariantLogpOp, NativeLinearLogpOp, VocabParallelLogprobOp, merge_tile_stats,
    tile_stats_reference)
