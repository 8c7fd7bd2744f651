from rl_kernel_b200.reference.embedding.embedding import (  # noqa: F401
    NativeEmbeddingOp, NativeLMHeadOp, embedding_grad_weight_reference)
