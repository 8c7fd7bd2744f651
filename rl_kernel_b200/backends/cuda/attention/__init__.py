from rl_kernel_b200.backends.cuda.attention.cp_comm import (AttentionCPBlockMetadata, AttentionCPCommunication,  # noqa: F401
                                                              AttentionCPCommunicationPlan,
                                                              AttentionCPCommunicationUnavailable,
                                                              AttentionCPMergedState, AttentionCPOutputShard,
                                                              AttentionCPPartialState, AttentionParallelSpec,
                                                              CPCommunicationBackend, CPCommunicationStatus,
                                                              CUDAAGRSAttentionCPCommunication,
                                                              P2PNCCLAttentionCPCommunication,
                                                              PeerMemoryAttentionCPCommunication,
                                                              sort_attention_cp_partial_states)
from rl_kernel_b200.backends.cuda.attention.deterministic_attn import (DeterministicAttentionCoreResult,  # noqa: F401
                                                                         DeterministicAttentionOp,
                                                                         RLKernelDeterministicAttentionCore)
from rl_kernel_b200.backends.cuda.attention.flash_attn import (FlashAttentionOp, StrictFlashAttention4Core,  # noqa: F401
                                                                 StrictFlashAttentionUnavailable)
from rl_kernel_b200.backends.cuda.attention.prefix_shared_attn import PrefixSharedAttentionOp  # noqa: F401
