"""Builds ``workloads/qwen3_8b.json`` (``python -m rl_kernel_b200.config.manifest_builder [--check]``).

The manifest is data, but most of it is regular: one representative case per (operator, fixture, profile).
Generating it keeps the three places that must agree -- operator specs, backend profiles and cases -- in one
table; ``--check`` (and a unit test) fail when the committed file differs from what this module produces.
"""
from __future__ import annotations

import argparse
import json
import sys

from rl_kernel_b200.config.workload import _MANIFEST_PATH, manifest_identity_hash, validate_manifest

H, I, HQ, HKV, D, V, VPAD = 4096, 12288, 32, 8, 128, 151936, 152576

FINGERPRINT = {"num_hidden_layers": 36, "hidden_size": H, "intermediate_size": I, "num_attention_heads": HQ,
               "num_key_value_heads": HKV, "head_dim": D, "vocab_size": V, "max_position_embeddings": 40960,
               "rope_theta": 1000000.0, "rms_norm_eps": 1e-06, "hidden_act": "silu", "swiglu": True,
               "tie_word_embeddings": False, "attention_bias": False, "qk_norm": True}

NODES = ["embedding", "input_layernorm", "qkv_proj", "qk_norm", "rope", "attention", "o_proj", "post_attention_layernorm",
         "gate_up_proj", "swiglu", "down_proj", "final_layernorm", "lm_head", "logprob"]

# chain node -> operator spec name
NODE_OPERATOR = {"embedding": "embedding", "input_layernorm": "rms_norm", "qkv_proj": "det_gemm", "qk_norm": "qk_norm",
                 "rope": "rope", "attention": "attention", "o_proj": "det_gemm", "post_attention_layernorm": "rms_norm",
                 "gate_up_proj": "det_gemm", "swiglu": "swiglu", "down_proj": "det_gemm", "final_layernorm": "rms_norm",
                 "lm_head": "lm_head", "logprob": "linear_logp"}

# operator spec -> (family, device class path, reference class path, algorithm source, algorithm property)
OPERATORS = {
    "det_gemm": ("gemm", "rl_engine.backends.cuda.gemm.det_gemm.DetGemmOp", "rl_engine.reference.gemm.det_gemm.NativeGemmOp",
                 "csrc/gemm/det_gemm_sm100.cu:det_gemm_kernel", "ordered_k_tcgen05_no_split_k"),
    "lm_head": ("gemm", "rl_engine.backends.cuda.embedding.lm_head.SM100LMHeadOp", "rl_engine.reference.embedding.lm_head.NativeLMHeadOp",
                "csrc/gemm/det_gemm_sm100.cu:det_gemm_kernel", "ordered_k_tcgen05_no_split_k"),
    "attention": ("attention", "rl_engine.backends.cuda.attention.deterministic_attn.DeterministicAttentionOp",
                  "rl_engine.reference.attention.standard_attn.NativeAttentionOp", "csrc/attention/attn_fwd_sm100.cu:attn_fwd_kernel",
                  "canonical_128_key_blocks_no_splitkv"),
    "kv_cache_attention": ("attention", "rl_engine.ops.attention.paged.paged_attention_block_table",
                           "rl_engine.reference.attention.kv_cache.NativeKVCacheAttnOp",
                           "csrc/attention/attn_fwd_sm100.cu:attn_fwd_kernel", "canonical_128_key_blocks_no_splitkv"),
    "prefix_shared_attention": ("attention", "rl_engine.backends.cuda.attention.prefix_shared_attn.PrefixSharedAttentionOp",
                                "rl_engine.validation.operators.operator_specs.GtestPrefixSharedAttentionOp",
                                "csrc/attention/attn_fwd_sm100.cu:attn_fwd_kernel", "group_rows_share_key_blocks"),
    "linear_logp": ("logprob", "rl_engine.backends.cuda.logprob.linear_logp.FusedLinearLogpSM100Op",
                    "rl_engine.reference.logprob.linear_logp.NativeLinearLogpOp", "csrc/gemm/det_gemm_sm100.cu:stats epilogue",
                    "vocab_tile128_ordered_merge"),
    "batch_invariant_logp": ("logprob", "rl_engine.backends.cuda.logprob.batch_invariant_logp.BatchInvariantLogpSM100Op",
                             "rl_engine.reference.logprob.batch_invariant_logp.NativeBatchInvariantLogpOp",
                             "csrc/logprob/logp.cu:logits_tile_stats_kernel", "vocab_tile128_ordered_merge"),
    "logp": ("logprob", "rl_engine.backends.cuda.logprob.logp.FusedLogpSM100Op", "rl_engine.reference.logprob.logp.NativeLogpOp",
             "csrc/logprob/logp.cu:logits_tile_stats_kernel", "vocab_tile128_ordered_merge"),
    "rms_norm": ("norm", "rl_engine.backends.cuda.norm.rmsnorm.RMSNormCudaOp", "rl_engine.reference.norm.rms_norm.NativeRMSNormOp",
                 "csrc/norm/rmsnorm.cu:rmsnorm_fwd_kernel", "row_local_fp32_statistics"),
    "qk_norm": ("norm", "rl_engine.backends.cuda.norm.rmsnorm.RMSNormCudaOp", "rl_engine.reference.norm.rms_norm.NativeRMSNormOp",
                "csrc/norm/rmsnorm.cu:qk_norm_rope_fwd_kernel", "row_local_fp32_statistics"),
    "rope": ("elementwise", "rl_engine.backends.cuda.rope.rope.RoPESM100Op", "rl_engine.reference.rope.rope.NativeRoPEOp",
             "csrc/rope/rope.cu:rope_kernel", "fp32_table_single_rounding"),
    "swiglu": ("elementwise", "rl_engine.backends.cuda.activation.swiglu.SwiGLUCudaOp", "rl_engine.reference.activation.swiglu.NativeSwiGLUOp",
               "csrc/activation/swiglu.cu:swiglu_fwd_kernel", "fp32_math_single_rounding"),
    "embedding": ("gather", "rl_engine.backends.cuda.embedding.embedding.SM100EmbeddingOp",
                  "rl_engine.reference.embedding.embedding.NativeEmbeddingOp", "csrc/embedding/embedding.cu:embedding_bwd_kernel",
                  "sorted_ids_one_warp_per_row"),
    "pack": ("layout", "rl_engine.ops.packing.PackOp", "rl_engine.reference.packing.pack.NativePackOp",
             "csrc/packing/pack.cu:move_rows_kernel", "row_major_cu_seqlens_order"),
    "grpo_loss": ("loss", "rl_engine.ops.loss.GRPOLossOp", "rl_engine.reference.loss.grpo_loss.NativeGRPOLossOp",
                  "csrc/loss/grpo_loss.cu:grpo_loss_kernel", "sequence_major_fixed_summation"),
    "sampling": ("sampling", "rl_engine.ops.sampling.api.SamplerBackend", "rl_engine.reference.sampling.policy.sample_from_logits",
                 "csrc/sampling/sampling.cu:sample_gumbel_kernel", "philox_keyed_gumbel_max"),
}

PRIMARY = [("s0", 11, 8, 100), ("s1", 16, 8, 900), ("s2", 13, 8, 1700), ("s3", 19, 8, 2500)]
LONG = [("l0", 150, 40, 7), ("l1", 260, 100, 11), ("l2", 129, 128, 13), ("l3", 300, 7, 17)]   # cross 128-token blocks


def _primary_sample(sid, n, p, base):
    return {"sample_id": sid, "seq_len": n, "prompt_len": p, "token_ids": [base + i for i in range(p)] + [base + 4000 + i for i in range(n - p)]}


def _shapes():
    """(case stem, operator spec, fixture, shape) for every representative case."""
    out = []
    for tag, m, fx in (("short-m8", 8, "short_full_model_seq8"), ("varlen-m59", 59, "primary_varlen"), ("long-m839", 839, "long_varlen"),
                       ("decode-m64", 64, "decode_context")):
        for name, k, n in (("qkv", H, (HQ + 2 * HKV) * D), ("o", HQ * D, H), ("gate-up", H, 2 * I), ("down", I, H)):
            out.append((f"gemm-{tag}-{name}-k{k}-n{n}", "det_gemm", fx, {"M": m, "K": k, "N": n}))
    out.append(("gemm-short-m8-lm-head-k4096-n151936", "lm_head", "short_full_model_seq8", {"M": 8, "K": H, "N": V}))
    out.append(("gemm-varlen-m59-lm-head-k4096-n151936", "lm_head", "primary_varlen", {"M": 59, "K": H, "N": V}))
    for stem, spec, fx, shape in (
        ("attn-short-prefill-gqa-b1-sq8-skv8", "attention", "short_full_model_seq8", {"mode": "prefill", "B": 1, "Sq": 8, "Skv": 8}),
        ("attn-varlen-prefill-gqa-b4", "attention", "primary_varlen", {"mode": "prefill", "B": 4, "Sq": [11, 16, 13, 19], "Skv": [11, 16, 13, 19]}),
        ("attn-long-prefill-gqa-b4", "attention", "long_varlen", {"mode": "prefill", "B": 4, "Sq": [150, 260, 129, 300], "Skv": [150, 260, 129, 300]}),
        ("attn-decode-gqa-b64-skv1024", "kv_cache_attention", "decode_context", {"mode": "decode", "B": 64, "Sq": 1, "Skv": 1024}),
        ("attn-chunked-prefill-gqa-b4-chunk7", "kv_cache_attention", "primary_varlen", {"mode": "chunked_prefill", "B": 4, "chunk": 7}),
        ("attn-prefix-shared-g8-p512", "prefix_shared_attention", "decode_context", {"mode": "decode", "B": 8, "G": 8, "Sq": 1, "Skv": 512}),
    ):
        out.append((stem, spec, fx, {**shape, "Hq": HQ, "Hkv": HKV, "D": D}))
    for stem, spec, fx, shape in (
        ("logp-short-vocab151936-t4", "linear_logp", "short_full_model_seq8", {"T": 4, "H": H, "V": V}),
        ("logp-varlen-vocab151936-t27", "linear_logp", "primary_varlen", {"T": 27, "H": H, "V": V}),
        ("logp-from-logits-varlen-t27", "batch_invariant_logp", "primary_varlen", {"T": 27, "V": V}),
        ("logp-indexed-long-t364", "logp", "long_varlen", {"T": 364, "V": V}),
    ):
        out.append((stem, spec, fx, shape))
    for spec, fam_shape in (("rms_norm", {"H": H}), ("qk_norm", {"heads": HQ + HKV, "D": D}), ("rope", {"heads": HQ + HKV, "D": D}),
                            ("swiglu", {"I": I}), ("embedding", {"V": V, "H": H})):
        for tag, t, fx in (("short-t8", 8, "short_full_model_seq8"), ("varlen-t59", 59, "primary_varlen")):
            out.append((f"{spec.replace('_', '-')}-{tag}", spec, fx, {"T": t, **fam_shape}))
    out.append(("pack-varlen-b4", "pack", "primary_varlen", {"B": 4, "S": 20, "H": H}))
    out.append(("grpo-loss-varlen-b4", "grpo_loss", "primary_varlen", {"B": 4, "S": 19, "group": 2}))
    out.append(("sampling-decode-b64-vocab151936", "sampling", "decode_context", {"B": 64, "V": V, "top_k": 0, "top_p": 1.0}))
    return out


def _case(stem, spec, fixture, shape, profile):
    family, device_path, ref_path, source, prop = OPERATORS[spec]
    backend, path = ("b200", device_path) if profile == "b200_bf16" else ("reference", ref_path)
    cid = f"{stem}-{backend}-v1"
    return {"case_id": cid, "family": family, "revision": 1, "fixture_id": fixture, "operator_spec": spec, "shape": shape,
            "expected_backend_id": backend, "expected_kernel_config_id": path, "actual_backend_id": backend,
            "actual_kernel_config_id": path, "provenance_status": "runtime_evidence_required", "algorithm_property": prop,
            "profile_ids": [profile], "architecture_identity": "full_qwen3_8b_dense",
            "provenance_evidence": {"kind": "runtime_execution_via_operator_specs",
                                    "registry": "rl_kernel_b200/validation/operators/operator_specs.py",
                                    "candidate_name": backend, "resolved_path": path,
                                    "algorithm_source": source if backend == "b200" else ref_path,
                                    "runtime_evidence_command": f"rlk verify --case-id {cid}"}}


def build() -> dict:
    cells = []
    for cid, mode, per, runs, prefill in (("B1-singleton_aggregate/full", "singleton_aggregate", 1, 4, "full"), ("BN/full", "batched", 4, 1, "full"),
                                          ("B1-singleton_aggregate/chunked", "singleton_aggregate", 1, 4, "chunked"),
                                          ("BN/chunked", "batched", 4, 1, "chunked")):
        cells.append({"cell_id": cid, "batch_mode": mode, "batch_size_per_run": per, "num_runs": runs, "prefill_mode": prefill,
                      "aggregation": {"order": "sample_ids", "denominator": "active_token_count_across_all_samples"}})
    profiles = {}
    for name, family, dtype, idx in (("b200_bf16", "b200", "bfloat16", 1), ("reference_fp32", "reference", "float32", 2)):
        profiles[name] = {"backend_family": family, "execution_dtype": dtype,
                          "operators": {node: OPERATORS[NODE_OPERATOR[node]][idx] for node in NODES}}
    raw = {
        "version": "2", "workload_id": "ws1-b200-v2", "seed": 20260812,
        "model_identity": {"model_id": "Qwen/Qwen3-8B", "config_fingerprint": FINGERPRINT, "padded_vocab_size": VPAD},
        "chain_semantics": {"nodes": NODES, "clip_interval": [0.8, 1.2], "kl_estimator": "k3_unbiased",
                            "loss_denominator": "active_token_count_across_all_samples",
                            "parity_thresholds": {"max_abs_dlogp": 0.06, "approx_kl0": 0.05, "clipfrac0": 0.0}},
        "stochastic_policy": {"dropout": 0, "sampling_is_seeded": True, "sampler": "philox_keyed_gumbel_max",
                              "key": ["seed", "step", "global_sequence", "position"]},
        "primary_matrix": {"N": 4, "batch_size_bn": 4, "sample_ids": [s[0] for s in PRIMARY], "sample_order_fixed": True,
                           "batch_permutation": {"enabled": True, "permutation": [2, 0, 3, 1]},
                           "chunk": {"chunk_size_tokens": 7, "require_ge_2_chunks": True, "non_divisible_case": True},
                           "long_chunk": {"chunk_size_tokens": 100}, "cells": cells},
        "fixtures": {
            "prompt_template": "ws1_fixed_token_fixture", "dtype_for_token_tensors": "int64",
            "position_ids": {"basis": "logical_zero_based_per_sample", "reset_after_pack_boundary": True},
            "attention_mask": {"active_value": 1, "padding_value": 0, "causal": True},
            "varlen_seq_lens": [s[1] for s in PRIMARY], "primary_prompt_len": 8,
            "padding": {"modes": ["right", "left"], "pad_token_id": 151643, "primary_padded_len": 20},
            "loss_mask": {"prompt_tokens_active": False, "completion_tokens_active": True},
            "samples": [_primary_sample(*s) for s in PRIMARY],
            "long_samples": [{"sample_id": sid, "seq_len": n, "prompt_len": p, "token_rule": {"base": 31 * b, "stride": b, "mod": V}}
                             for sid, n, p, b in LONG],
            "short_full_model_fixture": {"fixture_id": "short_full_model_seq8", "seq_len": 8, "prompt_len": 4,
                                         "token_ids": [310, 311, 312, 313, 410, 411, 412, 413]},
            "decode_context": {"fixture_id": "decode_context", "batch": 64, "context_len": 1024, "page_size": 128},
        },
        "logical_identity": {"key": ["sample_id", "token_position"], "compare": "raw_bits_for_invariance_tolerance_for_accuracy"},
        "capabilities": {"packing": True, "chunked_prefill": True, "left_padding": True, "paged_kv": True, "cuda_graph_decode": True},
        "backend_profiles": profiles,
        "representative_cases": [_case(*row, profile) for row in _shapes() for profile in ("b200_bf16", "reference_fp32")],
        "provenance_boundary": "a case is evidence only when `rlk verify --case-id` ran its operator spec on the named backend",
    }
    raw["fixture_identity_sha256"] = manifest_identity_hash(raw)
    validate_manifest(raw)
    return raw


def render() -> str:
    return json.dumps(build(), indent=1, sort_keys=False) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--check", action="store_true", help="fail if the committed manifest differs")
    a = ap.parse_args(argv)
    text = render()
    if a.check:
        same = _MANIFEST_PATH.exists() and _MANIFEST_PATH.read_text() == text
        print("manifest is up to date" if same else "manifest differs from the builder", file=sys.stderr)
        return 0 if same else 1
    _MANIFEST_PATH.write_text(text)
    print(f"wrote {_MANIFEST_PATH} ({len(build()['representative_cases'])} cases)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
