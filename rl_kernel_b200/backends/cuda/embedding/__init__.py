from rl_kernel_b200.backends.cuda.embedding.embedding import SM90EmbeddingOp, SM100EmbeddingOp  # noqa: F401
from rl_kernel_b200.backends.cuda.embedding.lm_head import SM90LMHeadOp, SM100LMHeadOp  # noqa: F401
