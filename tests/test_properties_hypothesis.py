"""Property tests (hypothesis) of the pieces whose correctness is a statement about ALL inputs: layout transforms keep
the logical tokens, restore maps invert them, the balanced tree does not care how leaves are spread over ranks, split-KV
plan sets of the reference path always align with themselves and never with a different chunking."""
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from rl_kernel_b200.config.workload import (LogicalBatch, LogicalSample, apply_chunking, apply_packing, apply_padding, permute_batch,  # noqa: E402
                                            restore_logical_order, restore_logical_order_from_padded, same_logical_multiset)
from rl_kernel_b200.contracts.operators.attention import AttentionContractError, validate_split_kv_plan_set_alignment  # noqa: E402
from rl_kernel_b200.distributed import balanced_tree_sum  # noqa: E402
from rl_kernel_b200.reference.attention.cp_attention import build_reference_split_kv_runtime_plan_set  # noqa: E402


@st.composite
def batches(draw):
    n = draw(st.integers(1, 5))
    samples = []
    for i in range(n):
        L = draw(st.integers(1, 40))
        ids = tuple(draw(st.lists(st.integers(0, 999), min_size=L, max_size=L)))
        samples.append(LogicalSample(f"s{i}", ids, draw(st.integers(0, L)), L))
    return LogicalBatch("prop", 0, tuple(samples))


@settings(max_examples=60, deadline=None)
@given(batches(), st.integers(1, 17), st.sampled_from(["left", "right"]), st.randoms(use_true_random=False))
def test_layout_transforms_keep_and_restore_the_logical_tokens(batch, chunk, side, rnd):
    truth = {(t.sample_id, t.token_position): t.token_id for s in batch.samples for t in s.tokens()}
    for layout in (apply_packing(batch), apply_chunking(batch, chunk_size=chunk)):
        assert restore_logical_order(layout, layout.physical_token_ids) == truth
        assert layout.num_tokens == len(truth) and sum(layout.segment_lengths) == len(truth)
        assert list(layout.cu_seqlens()) == sorted(layout.cu_seqlens()) and layout.cu_seqlens()[-1] == len(truth)
        assert sum(layout.physical_loss_mask) == batch.active_token_count()
    chunked = apply_chunking(batch, chunk_size=chunk)
    assert all(n <= chunk for n in chunked.segment_lengths)
    assert list(chunked.position_ids()) == [p for s in batch.samples for p in range(s.seq_len)]      # chunks of a sample stay in order
    padded = apply_padding(batch, pad_side=side, padded_len=max(s.seq_len for s in batch.samples) + 3)
    assert restore_logical_order_from_padded(padded, padded.physical_token_ids) == truth
    for b, s in enumerate(batch.samples):
        mask = padded.physical_attention_mask[b]
        assert sum(mask) == s.seq_len and (mask[0] == 0 if side == "left" else mask[-1] == 0)
        assert [p for p, m in zip(padded.physical_position_ids[b], mask) if m] == list(range(s.seq_len))
    perm = list(range(len(batch.samples)))
    rnd.shuffle(perm)
    shuffled = permute_batch(batch, perm)
    assert same_logical_multiset(shuffled, batch) and same_logical_multiset(shuffled, batch, active_only=False)
    assert restore_logical_order(apply_packing(shuffled), apply_packing(shuffled).physical_token_ids) == truth


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 2 ** 31 - 1), st.sampled_from([torch.bfloat16, torch.float32]), st.integers(1, 33))
def test_balanced_tree_is_the_same_function_however_the_leaves_are_grouped(seed, dtype, n):
    g = torch.Generator().manual_seed(seed)
    leaves = [(torch.randn(n, generator=g) * 10 ** float(torch.randint(-2, 3, (1,), generator=g))).to(dtype) for _ in range(8)]
    whole = balanced_tree_sum(leaves, dtype)
    for ranks in (2, 4, 8):                                        # each "rank" reduces its own leaves first, the ranks are combined by the same tree
        per = 8 // ranks
        partial = [balanced_tree_sum(leaves[r * per:(r + 1) * per], dtype) for r in range(ranks)]
        assert torch.equal(balanced_tree_sum(partial, dtype), whole)
    ints = [torch.randint(-1000, 1000, (n,), generator=g) for _ in range(4)]
    assert torch.equal(balanced_tree_sum(ints), sum(ints))


@settings(max_examples=40, deadline=None)
@given(st.lists(st.integers(8, 600), min_size=1, max_size=3), st.sampled_from([1, 2]), st.sampled_from([1, 2, 4]),
       st.sampled_from([None, 16, 100]), st.sampled_from([None, 16, 64]))
def test_reference_split_kv_plan_sets_align_only_with_the_same_chunking(totals, tp, cp, chunk_a, chunk_b):
    a = build_reference_split_kv_runtime_plan_set(totals, tp_world_size=tp, cp_world_size=cp, kv_chunk_size=chunk_a)
    assert len(a.entries) == len(totals) * tp * cp * cp
    validate_split_kv_plan_set_alignment(a, a)
    for e in a.entries:                                            # every plan tiles exactly its owner's range
        lo, hi = e.expected_kv_range
        assert e.execution.boundaries[0][0] == lo and e.execution.boundaries[-1][1] == hi
        assert all(x[1] == y[0] for x, y in zip(e.execution.boundaries, e.execution.boundaries[1:]))
    b = build_reference_split_kv_runtime_plan_set(totals, tp_world_size=tp, cp_world_size=cp, kv_chunk_size=chunk_b)
    if chunk_a == chunk_b:
        validate_split_kv_plan_set_alignment(a, b)
    else:
        with pytest.raises(AttentionContractError):
            validate_split_kv_plan_set_alignment(a, b)
