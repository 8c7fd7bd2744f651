"""Tensor parallelism simulated in one process (K split into shards, shards combined): the canonical tree gives the bits
of one rank at every TP degree and a plain left fold over eight shards does not -- the negative control that shows the
tree is what carries the invariance.  And the deterministic collective over a recording stand-in for torch.distributed:
what goes over the transport, in which order, and what a mismatching peer causes."""
import types

import pytest
import torch

from rl_kernel_b200.distributed import balanced_tree_sum
from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference

BF = torch.bfloat16


def _case(seed=0, M=9, K=1024, N=24):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(M, K, generator=g) * 2).to(BF), torch.randn(N, K, generator=g).to(BF)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_row_parallel_gemm_is_tp_invariant_with_the_canonical_tree(tp):
    x, w = _case()
    one = det_gemm_reference(x, w, nchunks=8)                      # one rank: eight canonical K chunks, balanced tree
    k = x.shape[1] // tp
    parts = [det_gemm_reference(x[:, r * k:(r + 1) * k], w[:, r * k:(r + 1) * k], nchunks=8 // tp) for r in range(tp)]
    assert torch.equal(balanced_tree_sum(parts, BF), one)          # the collective continues the tree the ranks started
    assert torch.equal(det_gemm_reference(x[:3], w, nchunks=8), one[:3])          # and rows do not depend on their neighbours


def test_left_fold_over_eight_shards_is_a_different_function():
    """Negative control: the same eight partial products added left to right (what a ring all-reduce or a chain of
    in-place adds does) round differently.  If this ever starts matching, the inputs are too tame to prove anything."""
    mismatches = 0
    for seed in range(4):
        x, w = _case(seed)
        k = x.shape[1] // 8
        leaves = [det_gemm_reference(x[:, r * k:(r + 1) * k], w[:, r * k:(r + 1) * k]) for r in range(8)]
        fold = leaves[0]
        for leaf in leaves[1:]:
            fold = (fold.float() + leaf.float()).to(BF)
        tree = det_gemm_reference(x, w, nchunks=8)
        assert torch.equal(balanced_tree_sum(leaves, BF), tree)
        mismatches += int((fold.view(torch.int16) != tree.view(torch.int16)).sum())
        assert (fold.float() - tree.float()).abs().max() < 0.05 * tree.float().abs().max()          # same value, other rounding
    assert mismatches > 0
    # unsplit fp32 accumulation over the whole K (one chunk) is yet another function than the 8-chunk tree
    x, w = _case(1)
    assert not torch.equal(det_gemm_reference(x, w, nchunks=1), det_gemm_reference(x, w, nchunks=8))


class _FakeDistributed:
    """Stand-in for ``torch.distributed`` seen from one rank of ``world``: peers' tensors come from ``peer_values``;
    every call is recorded."""

    def __init__(self, world: int, rank: int, peer_values=None, peer_signatures=None):
        self.world, self.rank, self.calls = world, rank, []
        self.peer_values, self.peer_signatures = peer_values or {}, peer_signatures
        self.group = types.SimpleNamespace(WORLD=None)

    def is_available(self):
        return True

    def is_initialized(self):
        return True

    def get_world_size(self, group=None):
        return self.world

    def get_rank(self, group=None):
        return self.rank

    def all_gather(self, out, t, group=None):
        self.calls.append(("all_gather", tuple(t.shape), str(t.dtype)))
        for r in range(self.world):
            out[r].copy_(t if r == self.rank else self.peer_values[r])

    def all_gather_into_tensor(self, out, t, group=None):
        self.all_gather(list(out.unbind(0)), t, group)

    def all_gather_object(self, out, obj, group=None):
        self.calls.append(("all_gather_object", obj))
        for r in range(self.world):
            out[r] = obj if (r == self.rank or self.peer_signatures is None) else self.peer_signatures[r]

    def all_reduce(self, t, group=None):
        self.calls.append(("all_reduce", tuple(t.shape)))

    def barrier(self, group=None):
        self.calls.append(("barrier",))


def _collective(fake):
    from rl_kernel_b200.distributed.algorithms import collectives as mod

    c = mod.TorchDistributedDeterministicCollective.__new__(mod.TorchDistributedDeterministicCollective)
    c._dist, c.group, c.world, c.rank = fake, None, fake.world, fake.rank
    import threading

    c._checked, c._check, c._lock = set(), True, threading.Lock()
    return c


def test_deterministic_collective_over_a_recording_transport():
    g = torch.Generator().manual_seed(3)
    parts = [torch.randn(64, generator=g).to(BF) for _ in range(4)]
    results = []
    for rank in range(4):
        fake = _FakeDistributed(4, rank, {r: parts[r] for r in range(4)})
        coll = _collective(fake)
        results.append(coll.all_reduce(parts[rank]))
        # a floating-point sum never travels as an all-reduce: one signature check, then one all-gather; the tree is local
        kinds = [c[0] for c in fake.calls]
        assert kinds == ["all_gather_object", "all_gather"], kinds
        coll.all_reduce(parts[rank])
        assert [c[0] for c in fake.calls][2:] == ["all_gather"]                     # the signature is checked once per (op, shape, dtype)
        n = torch.ones(3, dtype=torch.long)
        coll.all_reduce_int_(n)
        assert fake.calls[-1] == ("all_reduce", (3,))                                # integers may: their sum has no order
    want = balanced_tree_sum(parts, BF)
    assert all(torch.equal(r, want) for r in results)                                # every rank holds the same bits
    rs = _collective(_FakeDistributed(4, 2, {r: parts[r] for r in range(4)})).reduce_scatter(parts[2])
    assert torch.equal(rs, want[32:48])


def test_mismatching_peer_signature_is_refused_before_data_moves():
    from rl_kernel_b200.distributed import CollectiveMismatchError

    t = torch.zeros(8, dtype=BF)
    mine = ("all_gather", (8,), "torch.bfloat16")
    fake = _FakeDistributed(2, 0, {1: t}, peer_signatures={1: ("all_gather", (16,), "torch.bfloat16")})
    with pytest.raises(CollectiveMismatchError, match="signature mismatch"):
        _collective(fake).all_gather(t)
    assert fake.calls == [("all_gather_object", mine)]                               # nothing but the check went out
    with pytest.raises(ValueError):
        balanced_tree_sum([t, t, t])                                                 # the tree needs a power of two
    ok = _FakeDistributed(2, 0, {1: t})
    c = _collective(ok)
    c._check = False
    c.all_gather(t)
    assert [k[0] for k in ok.calls] == ["all_gather"]                                # checks can be switched off for the hot path
