"""Weight-sync bridge lifecycle on CPU: manifests, checksums, monotonic versions, rejection keeps the
previous version, shared memory across processes."""
import multiprocessing as mp

import pytest
import torch

from rl_engine.integrations.common.weights import (LocalTensorCopyBridge, SharedMemoryTensorBridge, UpdateState,
                                                   WeightInstallAdapter, WeightPublisher, WeightSyncError,
                                                   WeightUpdateManifest, reshard_blocks)
from rl_engine.integrations.engines.rollout.interface import RolloutExecutor


def _state(seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"a.weight": torch.randn(8, 4, generator=g).bfloat16(), "b.weight": torch.randn(16, generator=g)}


def test_local_bridge_lifecycle_and_rollback():
    bridge = LocalTensorCopyBridge()
    installed = {}
    ex = RolloutExecutor(bridge, WeightInstallAdapter(lambda t, m: installed.update({k: v.clone() for k, v in t.items()})))
    pub = WeightPublisher(bridge)
    m1 = pub.publish(_state(1), 1)
    assert WeightUpdateManifest.from_json(m1.to_json()).tensors["a.weight"].sha256 == m1.tensors["a.weight"].sha256
    assert ex.update_weights(m1)["status"] == "acknowledged" and ex.weight_version == 1
    # a failing install rejects the update and keeps version 1
    bad = RolloutExecutor(bridge, WeightInstallAdapter(lambda t, m: (_ for _ in ()).throw(RuntimeError("boom"))))
    bad.weight_version = 1
    m2 = pub.publish(_state(2), 2)
    r = bad.update_weights(m2)
    assert r["status"] == "rejected" and "boom" in r["reason"] and bad.weight_version == 1
    assert bridge.state(m2.update_id) == UpdateState.REJECTED
    m3 = pub.publish(_state(3), 3)
    assert ex.update_weights(m3)["status"] == "acknowledged"
    assert bridge.state(m1.update_id) == UpdateState.RELEASED          # previous update released on ack
    assert torch.equal(installed["a.weight"], _state(3)["a.weight"])
    with pytest.raises(WeightSyncError):
        pub.publish(_state(4), 3)                                       # version must increase
    stale = WeightUpdateManifest.from_json(m1.to_json())
    assert ex.update_weights(stale)["status"] == "rejected"


def test_checksum_mismatch_is_rejected():
    bridge = LocalTensorCopyBridge()
    m = bridge.publish(_state(), 1)
    bridge._payload[m.update_id]["a.weight"][0, 0] += 1                  # tamper after publishing
    ex = RolloutExecutor(bridge, WeightInstallAdapter(lambda t, m: None))
    r = ex.update_weights(m)
    assert r["status"] == "rejected" and "checksum" in r["reason"]


def test_unsupported_layout():
    bridge = LocalTensorCopyBridge()
    with pytest.raises(WeightSyncError):
        bridge.publish(_state(), 1, {"layout": "pipeline-sharded"})
    with pytest.raises(WeightSyncError):
        bridge.publish(_state(), 2, {"node_count": 2})


def _consumer(manifest_json, q):
    b = SharedMemoryTensorBridge()
    m = WeightUpdateManifest.from_json(manifest_json)
    t = b.import_update(m)
    q.put({k: v.float().sum().item() for k, v in t.items()})
    for seg in b._segments.values():
        seg.close()


def test_shared_memory_bridge_across_processes():
    bridge = SharedMemoryTensorBridge()
    st = _state(5)
    m = bridge.publish(st, 1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_consumer, args=(m.to_json(), q))
    p.start()
    got = q.get(timeout=120)
    p.join(120)
    assert got == {k: v.float().sum().item() for k, v in st.items()}
    bridge.release(m.update_id)
    bridge.close()


def test_reshard_block_lists_cover_destination():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.engine import PackedParams

    spec = Qwen3DenseSpec.scaled(layers=1, hidden=128, ffn=256, q_heads=4, kv_heads=2, head_dim=128, vocab=512)
    cpu = torch.device("cpu")
    full = PackedParams(spec, 0, 1, cpu)
    full.flat.copy_(torch.arange(full.numel, dtype=torch.float32).bfloat16())
    # emulate the push on the host: TP1 source -> two TP2 destination shards, and back
    dsts = [PackedParams(spec, r, 2, cpu) for r in range(2)]
    for i, d in enumerate(dsts):
        for (so, do, sp, dp, rows, rb, mask) in reshard_blocks(full, d, i):
            src8, dst8 = full.flat.view(torch.uint8), d.flat.view(torch.uint8)
            for r in range(rows):
                dst8[do + r * dp: do + r * dp + rb] = src8[so + r * sp: so + r * sp + rb]
    want = [PackedParams(spec, r, 2, cpu) for r in range(2)]
    from rl_kernel_b200.models.qwen3.weights import Qwen3DenseWeights
    hf = full.export_local()
    for r in range(2):
        want[r].load(Qwen3DenseWeights({k: v.clone() for k, v in hf.items()}, "x"))
        assert torch.equal(want[r].flat, dsts[r].flat)
