from rl_kernel_b200.backends.cuda.ffn.ffn import (BACKEND_ID, Qwen3FFNOp, qwen3_ffn, qwen3_ffn_packed_inference,  # noqa: F401
                                                  register_packed_inference_observer)
