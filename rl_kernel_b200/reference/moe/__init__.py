from rl_kernel_b200.reference.moe.moe import (moe_dispatch_plan_reference, moe_ffn_reference,  # noqa: F401
                                              router_topk_reference)
