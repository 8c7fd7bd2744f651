"""Weight-sync bridge lifecycle on CPU: manifests, checksums, monotonic versions, rejection keeps the
previous version, shared memory across processes."""
import multiprocessing as mp

import pytest
import torch

from rl_engine.integrations.common.weights import (CallableInstallAdapter, LocalTensorCopyBridge,
                                                   SharedMemoryTensorBridge, TensorDescriptor, UpdateState,
                                                   VLLMCheckpointWeightReloadAdapter, VLLMCUDAVMMExternalStorageAdapter,
                                                   VLLMInProcessWeightReloadAdapter, VLLMIPCWeightUpdateRequestBuilder,
                                                   VLLMWeightInstallAdapter, WeightBridgeError,
                                                   WeightBridgeUnavailableError, WeightLayout,
                                                   WeightManifestValidationError, WeightPublisher, WeightSyncError,
                                                   WeightUpdateManifest, WeightUpdateRejectedError, make_weight_bridge,
                                                   reshard_blocks)
from rl_engine.integrations.engines.rollout.interface import RolloutExecutor


def _state(seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"a.weight": torch.randn(8, 4, generator=g).bfloat16(), "b.weight": torch.randn(16, generator=g)}


def test_local_bridge_lifecycle_and_rollback():
    bridge = LocalTensorCopyBridge()
    installed = {}
    ex = RolloutExecutor(weight_bridge=bridge, weight_install_adapter=CallableInstallAdapter(
        lambda m, t: installed.update({k: v.clone() for k, v in t.items()})))
    pub = WeightPublisher(bridge)
    m1 = pub.publish(_state(1), 1)
    assert WeightUpdateManifest.from_json(m1.to_json()) == m1
    assert m1.tensor_count == 2 and m1.total_nbytes == 8 * 4 * 2 + 16 * 4
    assert m1.tensors["a.weight"].name == "a.weight" and m1.tensors["a.weight"].dtype == "torch.bfloat16"
    assert ex.try_update_weights(m1)["status"] == "acknowledged" and ex.weight_version == 1
    assert bridge.active_weight_version == 1 and bridge.active_update_id == m1.update_id
    # a failing install rejects the update and keeps version 1
    def boom(m, t):
        raise RuntimeError("boom")
    bad = RolloutExecutor(weight_bridge=bridge, weight_install_adapter=CallableInstallAdapter(boom))
    bad.weight_version = 1
    m2 = pub.publish(_state(2), 2)
    r = bad.try_update_weights(m2)
    assert r["status"] == "rejected" and "boom" in r["reason"] and bad.weight_version == 1
    assert bridge.update_status(m2.update_id) == UpdateState.REJECTED
    with pytest.raises(RuntimeError, match="boom"):
        bad.update_weights(pub.publish(_state(2), 3))                   # the raising form of the same call
    m3 = pub.publish(_state(3), 4)
    assert ex.try_update_weights(m3)["status"] == "acknowledged"
    assert bridge.update_status(m1.update_id) == UpdateState.RELEASED   # the superseded update is released
    assert torch.equal(installed["a.weight"], _state(3)["a.weight"])
    with pytest.raises(WeightManifestValidationError):
        pub.publish(_state(4), 4)                                       # version must increase
    assert ex.try_update_weights(m1)["status"] == "rejected"            # stale and released
    with pytest.raises(WeightUpdateRejectedError):
        bridge.acknowledge(pub.publish(_state(5), 5).update_id)         # no acknowledge before an import
    assert issubclass(WeightManifestValidationError, WeightBridgeError) and WeightSyncError is WeightBridgeError


def test_checksum_mismatch_is_rejected():
    bridge = LocalTensorCopyBridge()
    m = bridge.publish(_state(), weight_version=1)
    bridge._updates[m.update_id].tensors["a.weight"][0, 0] += 1          # tamper after publishing
    ex = RolloutExecutor(weight_bridge=bridge)
    r = ex.try_update_weights(m)
    assert r["status"] == "rejected" and "checksum" in r["reason"]


def test_unsupported_layouts_and_factory():
    bridge = make_weight_bridge("local-clone", source_worker="w7", source_rank=3)
    m = bridge.publish(torch.nn.Linear(4, 2), weight_version=1)          # a module publishes its state_dict
    assert m.source_worker == "w7" and m.source_rank == 3 and set(m.tensors) == {"weight", "bias"}
    assert m.metadata["layout"]["kind"] == "full-state"
    with pytest.raises(WeightBridgeUnavailableError):
        bridge.publish(_state(), weight_version=2, metadata={"layout": {"kind": "pipeline-sharded"}})
    with pytest.raises(WeightBridgeUnavailableError):
        bridge.publish(_state(), weight_version=2, metadata={"layout": {"kind": "full-state", "tensor_parallel_size": 2}})
    with pytest.raises(WeightBridgeUnavailableError):
        bridge.publish(_state(), weight_version=2, metadata={"layout": {"node_count": 2}})
    with pytest.raises(WeightManifestValidationError):
        WeightLayout(world_size=2, rank=2).validate_supported()
    assert isinstance(make_weight_bridge("shm"), SharedMemoryTensorBridge)
    with pytest.raises(WeightBridgeUnavailableError):
        make_weight_bridge("rdma")
    with pytest.raises(WeightBridgeUnavailableError):
        make_weight_bridge("carrier-pigeon")


def test_manifest_with_the_reference_field_names_round_trips():
    """A manifest serialised with exactly the reference's fields (TensorDescriptor.name, dtype with
    the ``torch.`` prefix, ``created_at``, layout as a mapping, no offset) loads, validates against a
    local update of the same content and serialises back to the same fields."""
    st = _state(9)
    bridge = LocalTensorCopyBridge(source_worker="local-training", source_rank=0)
    ours = bridge.publish(st, weight_version=5)
    ref_style = {
        "update_id": ours.update_id, "source_worker": "local-training", "source_rank": 0, "weight_version": 5,
        "transport": "local-clone", "created_at": ours.created_at,
        "metadata": {"layout": {"kind": "full-state", "world_size": 1, "rank": 0, "tensor_parallel_size": 1,
                                "data_parallel_size": 1, "zero_stage": 0, "node_count": 1, "rdma_enabled": False}},
        "tensors": {k: {"name": k, "shape": list(v.shape), "dtype": str(v.dtype), "stride": list(v.stride()),
                        "device": "cpu", "numel": v.numel(), "nbytes": v.numel() * v.element_size(),
                        "sha256": ours.tensors[k].sha256} for k, v in st.items()},
    }
    m = WeightUpdateManifest.from_dict(ref_style)
    assert m == ours
    got = bridge.import_update(m)
    assert all(torch.equal(got[k], st[k]) for k in st)
    back = __import__("json").loads(m.to_json())
    for k in st:
        for f in ("name", "shape", "dtype", "stride", "device", "numel", "nbytes", "sha256"):
            assert back["tensors"][k][f] == ref_style["tensors"][k][f]
    assert back["created_at"] == ref_style["created_at"] and back["metadata"]["layout"] == ref_style["metadata"]["layout"]
    d = TensorDescriptor.from_tensor("x", torch.zeros(2, 3))
    assert (d.dtype, d.shape, d.stride, d.offset) == ("torch.float32", (2, 3), (3, 1), 0) and len(d.sha256) == 64


class _FakeVLLM:
    def __init__(self):
        self.calls = []

    def update_weights(self, request):
        self.calls.append(("update_weights", request))

    def collective_rpc(self, method, kwargs=None):
        self.calls.append((method, kwargs))


def test_vllm_install_adapters_against_a_fake_engine():
    bridge = LocalTensorCopyBridge()
    m = bridge.publish(_state(3), weight_version=1)
    t = bridge.import_update(m)
    eng = _FakeVLLM()
    with pytest.raises(WeightBridgeUnavailableError):
        VLLMWeightInstallAdapter(eng).install(m, t)                      # update_weights needs a request builder
    ad = VLLMWeightInstallAdapter(eng, request_builder=lambda mm, tt: {"n": len(tt)})
    ad.install(m, t)
    assert eng.calls[-1] == ("update_weights", {"n": 2}) and ad.active_weight_version == 1
    ad.release(m.update_id)
    assert ad.active_update_id is None
    seen = {}
    VLLMWeightInstallAdapter(object(), install_callable=lambda mm, tt: seen.update(tt)).install(m, t)
    assert set(seen) == set(t)
    # in-process reload: named tensors through collective_rpc("reload_weights")
    ip = VLLMInProcessWeightReloadAdapter(eng, target_dtype=torch.float32, synchronize_cuda=False)
    ip.install(m, t)
    method, kw = eng.calls[-1]
    assert method == "reload_weights" and [n for n, _ in kw["weights_iterator"]] == list(m.tensors)
    assert all(w.dtype == torch.float32 for _, w in kw["weights_iterator"]) and kw["is_checkpoint_format"] is True
    with pytest.raises(WeightManifestValidationError):
        ip.install(m, {"a.weight": t["a.weight"]})
    # checkpoint reload: only a path crosses the RPC boundary
    ck = VLLMCheckpointWeightReloadAdapter(eng, synchronize_cuda=False)
    with pytest.raises(WeightBridgeUnavailableError):
        ck.install(m, t)
    ck = VLLMCheckpointWeightReloadAdapter(eng, weights_path_resolver=lambda mm, tt: f"/ckpt/v{mm.weight_version}",
                                           synchronize_cuda=False)
    ck.install(m, t)
    assert eng.calls[-1] == ("reload_weights", {"weights_path": "/ckpt/v1", "is_checkpoint_format": True})
    # IPC request builder (CPU tensors are refused; with fake handles the public request shape comes out)
    rb = VLLMIPCWeightUpdateRequestBuilder(reduce_tensor_fn=lambda w: ("handle", tuple(w.shape)), gpu_uuid="GPU-x")
    with pytest.raises(WeightBridgeUnavailableError):
        rb(m, t)
    # external storage: the model's parameters alias the imported tensors until release
    model = torch.nn.ModuleDict({"a": torch.nn.Linear(4, 8, bias=False).bfloat16()})
    mm = bridge.publish({"a.weight": _state(3)["a.weight"]}, weight_version=2)
    tt = bridge.import_update(mm)
    before = model["a"].weight.data
    es = VLLMCUDAVMMExternalStorageAdapter(model)
    es.install(mm, tt)
    assert model["a"].weight.data_ptr() == tt["a.weight"].data_ptr()
    es.release(mm.update_id)
    assert model["a"].weight.data_ptr() == before.data_ptr()


def _consumer(manifest_json, q):
    b = SharedMemoryTensorBridge()
    m = WeightUpdateManifest.from_json(manifest_json)
    t = b.import_update(m)
    q.put({k: v.float().sum().item() for k, v in t.items()})
    del t
    b.release(m.update_id)


def test_shared_memory_bridge_across_processes():
    bridge = SharedMemoryTensorBridge()
    st = _state(5)
    m = bridge.publish(st, weight_version=1)
    assert m.metadata["rl_kernel_bridge"]["format"] == "posix-shm-v1"
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
