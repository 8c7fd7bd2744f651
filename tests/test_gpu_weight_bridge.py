"""Device transports of the weight bridge on one GPU: the cuda-vmm transport across two processes
(the importer maps the publisher's allocation and reads the same bytes) and its install path that
makes a model's parameters alias the imported tensors."""
import multiprocessing as mp

import pytest
import torch

pytestmark = pytest.mark.gpu


def _vmm_consumer(manifest_json, q):
    import torch

    from rl_kernel_b200.integrations.common.weights import CUDAVMMTensorBridge, WeightUpdateManifest

    try:
        b = CUDAVMMTensorBridge(device="cuda:0")
        m = WeightUpdateManifest.from_json(manifest_json)
        t = b.import_update(m)                       # descriptors and checksums are verified here
        sums = {k: v.float().sum().item() for k, v in t.items()}
        ptr_inside = all(v.is_cuda for v in t.values())
        b.acknowledge(m.update_id)
        del t
        b.release(m.update_id)
        q.put(("ok", sums, ptr_inside))
    except Exception as exc:  # noqa: BLE001 - reported to the parent
        q.put(("error", f"{type(exc).__name__}: {exc}", False))


def test_cuda_vmm_bridge_across_processes():
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.integrations.common.weights import CUDAVMMTensorBridge, VLLMCUDAVMMExternalStorageAdapter

    dev = torch.device("cuda:0")
    with torch.cuda.device(dev):
        if not ext.load().rlk_vmm_supported():
            pytest.skip("no POSIX-descriptor virtual memory on this driver")
    g = torch.Generator(device="cuda").manual_seed(3)
    state = {"a.weight": torch.randn(257, 129, device=dev, generator=g).bfloat16(),
             "b.weight": torch.randn(1000, device=dev, generator=g),
             "c.ids": torch.arange(77, device=dev, dtype=torch.int64)}
    bridge = CUDAVMMTensorBridge(device=dev, source_worker="trainer", source_rank=0)
    m = bridge.publish(state, weight_version=1)
    info = m.metadata["rl_kernel_bridge"]
    assert info["format"] == "cuda-vmm-fd-v1" and info["mapped_nbytes"] >= m.total_nbytes
    assert all(d.offset % 256 == 0 and d.device == "cuda:0" for d in m.tensors.values())
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_vmm_consumer, args=(m.to_json(), q))
    p.start()
    status, sums, on_gpu = q.get(timeout=300)
    p.join(120)
    assert status == "ok", sums
    assert on_gpu and sums == {k: v.float().sum().item() for k, v in state.items()}
    # same-process import aliases the allocation; the external-storage adapter points a model at it
    t = bridge.import_update(m)
    assert t["a.weight"].data_ptr() == bridge.debug_tensor_data_ptrs(m.update_id)["a.weight"]
    model = torch.nn.ModuleDict({"a": torch.nn.Linear(129, 257, bias=False, device=dev, dtype=torch.bfloat16)})
    ad = VLLMCUDAVMMExternalStorageAdapter(model, name_map=lambda n: n)
    sub = bridge.publish({"a.weight": state["a.weight"]}, weight_version=2)
    ts = bridge.import_update(sub)
    ad.install(sub, ts)
    assert model["a"].weight.data_ptr() == ts["a.weight"].data_ptr() and torch.equal(model["a"].weight.data, state["a.weight"])
    ad.release(sub.update_id)
    del t, ts
    bridge.close()
    torch.cuda.synchronize()
