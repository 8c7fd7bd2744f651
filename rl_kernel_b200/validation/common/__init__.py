"""Testing helpers for RL-shaped kernel validation (parity: rl_engine/validation/common/__init__.py:6-113)."""
from rl_kernel_b200.config.workload import (LogicalBatch, PhysicalLayout, WorkloadError, WS1Manifest, apply_chunking, apply_packing,
                                            apply_padding, build_logical_batch, fixture_hash, load_manifest, reference_payload,
                                            restore_logical_order, restore_logical_order_from_padded)
from rl_kernel_b200.reference.definitions import (active_token_count, compute_policy_ratio, compute_reference_kl, masked_mean,
                                                  masked_sum, selected_logprobs_reference, summarize_kernel_drift)
from rl_kernel_b200.validation.common.attention_comparison import (AttentionComparisonInputs, AttentionComparisonReport,
                                                                   AttentionPathDrift, AttentionPathResult,
                                                                   DecodeAttentionInputs, DecodeKVCacheMetadata, DriftStats,
                                                                   TransformerEngineUnavailable, compare_decode_kv_replay,
                                                                   compare_single_gpu_attention,
                                                                   compare_single_gpu_rope_attention,
                                                                   decode_kv_cache_fingerprint,
                                                                   decode_prefix_cache_fingerprint,
                                                                   decode_rope_identity_fingerprint,
                                                                   run_chunked_query_attention,
                                                                   run_decode_full_prefill_reference, run_decode_kv_replay,
                                                                   run_decode_strict_shared_core, run_device_attention,
                                                                   run_full_attention, run_fused_like_rope_attention,
                                                                   run_paged_kv_attention, run_strict_shared_core_attention,
                                                                   run_strict_shared_core_chunked_attention,
                                                                   run_strict_shared_core_paged_layout_attention,
                                                                   run_unfused_rope_attention,
                                                                   transformer_engine_context_parallel_available)
from rl_kernel_b200.validation.common.logprob_drift import LogprobDriftStats, summarize_logprob_drift
from rl_kernel_b200.validation.common.rl_batch import SyntheticRLBatch, SyntheticRLKernelBatch, make_synthetic_rl_kernel_batch

__all__ = [n for n in dir() if not n.startswith("_")]
