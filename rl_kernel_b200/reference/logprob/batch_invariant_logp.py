"""Batch-invariant selected log-prob from materialised logits in PyTorch
(parity: NativeBatchInvariantLogpOp, rl_engine/reference/logprob/batch_invariant_logp.py:9).

The row reduction follows the 128-id tile contract of ``tile_logp`` -- fixed per-tile order, tiles
merged in ascending order -- so a row's value never depends on the other rows of the call, on how
the batch was chunked, permuted or padded, or on how many vocabulary shards computed it."""
from rl_kernel_b200.reference.logprob.tile_logp import (TILE, NativeBatchInvariantLogpOp, merge_tile_stats,  # noqa: F401
                                                        tile_stats_reference)

__all__ = ["NativeBatchInvariantLogpOp", "TILE", "merge_tile_stats", "tile_stats_reference"]
