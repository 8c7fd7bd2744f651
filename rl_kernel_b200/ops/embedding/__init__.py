from rl_kernel_b200.ops.embedding.canonical_embedding import EmbeddingOp, embedding  # noqa: F401
from rl_kernel_b200.ops.embedding.canonical_lm_head import LMHeadOp, lm_head_logits  # noqa: F401
